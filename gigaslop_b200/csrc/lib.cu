// libgigaslop_b200 is built as one translation unit so that the device status
// word and the inline PTX helpers are shared without relocatable device code.
#include "quant.cu"
#include "gemm.cu"
#include "lstm.cu"
#include "factored.cu"
#include "mx_gemm.cu"
#include "probe.cu"
#include "capi.cu"
