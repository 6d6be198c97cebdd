"""Oracle: MXFP8 block scaling (E4M3 elements, one E8M0 scale per 32 elements).

Test infrastructure only.  **Parity unpinned**: the reference ships only the
interface of its MXFP8 kernel (``fly/export_fp8_dual_gemm_silu_mxfp8.py:145-236``;
the kernel module it imports at ``:31`` is absent), so there is no reference
function, test or golden vector.  The scale rule below is the OCP
Microscaling v1.0 default and is the rule the device kernels implement:

    e      = biased fp32 exponent of max|v| over the 32-element block
    byte   = clamp(e - 8, 0, 254)            # E8M0, value 2**(byte-127); 8 = emax(E4M3)
    q[i]   = e4m3_rn_satfinite(v[i] * 2**(127-byte))

so the scaled block maximum lands in [256, 512) and values above 448
saturate.  An all-zero block gets byte 0.
"""
import torch

BLOCK = 32


def e8m0_decode(b):
    """uint8 -> fp32 ``2**(b-127)`` (exact; 0xff would be NaN and is never produced)."""
    e = b.to(torch.int32) - 127
    return torch.ldexp(torch.ones(e.shape, dtype=torch.float32), e)


def mx_block_quantize(v):
    """fp32 ``[..., K]`` (K % 32 == 0) -> (float8_e4m3fn ``[..., K]``, uint8 ``[..., K/32]``)."""
    v = v.float().contiguous()
    shp = v.shape
    blk = v.reshape(*shp[:-1], shp[-1] // BLOCK, BLOCK)
    amax = blk.abs().amax(dim=-1)
    e = (amax.view(torch.int32) >> 23) & 0xFF
    byte = (e - 8).clamp(0, 254)
    inv = torch.ldexp(torch.ones_like(amax), 127 - byte)
    q = (blk * inv.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q.reshape(shp), byte.to(torch.uint8)


def mx_dequantize(q, s):
    """Inverse of :func:`mx_block_quantize` (exact in fp32)."""
    shp = q.shape
    blk = q.float().reshape(*shp[:-1], shp[-1] // BLOCK, BLOCK)
    return (blk * e8m0_decode(s).unsqueeze(-1)).reshape(shp)


def mx_gemm_ref(Aq, As, Wq, Ws):
    """Block-scaled GEMM ``D[m,n] = sum_k A[m,k]*W[n,k]`` on dequantised operands,
    float64 accumulation (what ``kind::mxf8f6f4`` computes up to fp32 summation order)."""
    return (mx_dequantize(Aq, As).double() @ mx_dequantize(Wq, Ws).double().T).float()


def mx_dual_silu_ref(Aq, As, Wgq, Wgs, Wuq, Wus):
    """SwiGLU on block-scaled operands: ``silu(A.Wg^T) * (A.Wu^T)`` in fp32."""
    g = mx_gemm_ref(Aq, As, Wgq, Wgs)
    u = mx_gemm_ref(Aq, As, Wuq, Wus)
    return g * torch.sigmoid(g) * u
