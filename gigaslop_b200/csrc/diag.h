// Diagnostic switches of the GEMM family.  They exist only in a library built with -DGSB200_DIAG (timing
// ablations and alternative code paths used while tuning; two of them produce wrong output by design), are not
// part of the public header, and the shipped library rejects their bits like any unknown flag.
#pragma once
#define GSB200_DIAG_FLAG_DIRECT_STORE 1      // epilogue stores straight from registers (no shared-memory staging, no TMA store)
#define GSB200_DIAG_FLAG_STREAMING 2         // stream both operands even when one of them could stay resident
#define GSB200_DIAG_FLAG_ABLATE_STORES 0x100    // output is NOT written: skip the epilogue's stores
#define GSB200_DIAG_FLAG_ABLATE_EPILOGUE 0x200  // output is NOT written: skip the epilogue body
#define GSB200_DIAG_FLAG_ABLATE_MAINLOOP 0x400  // accumulators are garbage: skip the loads and the MMAs
#ifdef GSB200_DIAG
#define GSB200_DIAG_FLAG_ABLATE_HALF_WARPS 0x800 // half of the output is NOT written: the epilogue warps of the second column half skip their body
#define GSB200_DIAG_FLAG_MASK 0xF03
#else
#define GSB200_DIAG_FLAG_MASK 0
#endif
