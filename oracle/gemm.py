"""Oracle: W8A8 / FP8 GEMMs and their fused epilogues (CPU, PyTorch).

Test infrastructure only.  Two kinds of function live here:

``*_ref``   the reference's own host reference, restated (dequantise to fp32,
            then fp32 matmul) -- the tolerance-checked oracle.
``*_exact`` / ``*_model``  the arithmetic the device kernels perform on the
            *exact* int32 accumulator, operation by operation, so that integer
            paths can be compared bit for bit and fp paths to ~1 ulp.
"""
import torch


def gemm_i32(A_i8, B_i8):
    """Exact int32 accumulators ``A[M,K] . B[N,K]^T``.

    Follows ``cute/ampere_gemm_i8.py:704-709`` (int32 ``torch.matmul`` on CPU,
    checked with atol=rtol=0 at ``:838-845``).
    """
    M, K = A_i8.shape
    if M > 16 and K % 8 == 0 and B_i8.shape[0] % 8 == 0:
        try:
            return torch._int_mm(A_i8.contiguous(), B_i8.t())
        except RuntimeError:
            pass
    return A_i8.to(torch.int32) @ B_i8.to(torch.int32).t()


def gemm_dequant_ref(A_i8, B_i8, scale_a, scale_b):
    """fp32 reference of the dequantising GEMM: dequantise first, then matmul.

    Follows ``cute/ampere_gemm_i8_rotary.py:493-495`` and the C++ host check
    ``cute/main.cpp:136-143``.
    """
    A_dq = A_i8.float() * scale_a[:, None]
    B_dq = B_i8.float() * scale_b[:, None]
    return A_dq @ B_dq.T


def gemm_dequant_exact(A_i8, B_i8, scale_a, scale_b):
    """Bit-exact model of the kernel epilogue: ``f16(f32(acc) * (sA[m]*sB[n]))``.

    The two scales are multiplied first and the product applied to the
    converted accumulator, as in ``cute/ampere_gemm_i8_quant_rmem.py:593-603,723-732``.
    """
    acc = gemm_i32(A_i8, B_i8).float()
    s = scale_a.float()[:, None] * scale_b.float()[None, :]
    return (acc * s).to(torch.float16)


def rope_tables(seqlen, rotary_half, head_dim, base=10000.0):
    """Canonical RoPE sin/cos tables ``[seqlen, rotary_half]`` fp32.

    Same formula as ``cute/test_gemm_i8_rotary_vs_openfish.py:67-72``.
    """
    inv_freq = 1.0 / (base ** (torch.arange(0, rotary_half).float() / head_dim * 2))
    t = torch.arange(seqlen).float()
    freqs = torch.outer(t, inv_freq)
    return freqs.sin().contiguous(), freqs.cos().contiguous()


def _rotate(C, sin_buf, cos_buf, nhead, head_dim, rotary_dim, seqlen):
    M = C.shape[0]
    rh = rotary_dim // 2
    out = C.clone()
    seq = torch.arange(M) % seqlen
    sin = sin_buf[seq]
    cos = cos_buf[seq]
    for hs in range(0, 2 * nhead * head_dim, head_dim):
        x0 = C[:, hs:hs + rh]
        x1 = C[:, hs + rh:hs + rotary_dim]
        out[:, hs:hs + rh] = x0 * cos - x1 * sin
        out[:, hs + rh:hs + rotary_dim] = x0 * sin + x1 * cos
    return out


def rotary_ref(A_i8, B_i8, scale_a, scale_b, sin_buf, cos_buf,
               nhead, head_dim, rotary_dim, seqlen):
    """fp32 reference of the QKV GEMM with rotary on the Q and K columns.

    Follows ``cute/ampere_gemm_i8_rotary.py:487-506``: dequantised fp32 matmul,
    then per head ``out[k] = x0*cos - x1*sin``, ``out[k+rh] = x0*sin + x1*cos``
    with the angle row ``m % seqlen``; V columns and columns past
    ``rotary_dim`` inside a head pass through.
    """
    C = gemm_dequant_ref(A_i8, B_i8, scale_a, scale_b)
    return _rotate(C, sin_buf, cos_buf, nhead, head_dim, rotary_dim, seqlen)


def fma_f32(a, b, c):
    """Correctly rounded fp32 fused multiply-add ``round(a*b + c)`` of float32 tensors.

    The product of two float32 is exact in float64; the sum is rounded to odd in
    float64 (TwoSum gives the discarded part), which makes the final rounding to
    float32 the same as rounding the exact value once."""
    p = a.double() * b.double()
    cd = c.double().expand_as(p)
    s = p + cd
    bb = s - p
    err = (p - (s - bb)) + (cd - bb)
    bits = s.contiguous().view(torch.int64)
    need = (err != 0) & ((bits & 1) == 0)
    step = torch.where((err > 0) == (s > 0), 1, -1)
    bits = torch.where(need, bits + step, bits)
    return bits.view(torch.float64).float()


def rotary_exact(A_i8, B_i8, scale_a, scale_b, sin_buf, cos_buf,
                 nhead, head_dim, rotary_dim, seqlen):
    """Model of the device epilogue on the exact int32 accumulator, rounding where the kernel rounds.

    Rotated columns: ``y = f32(acc)*sB[n]``, ``C = sA[m]*cos``, ``S = sA[m]*sin`` (each one
    rounded fp32 product), then ``out0 = fma(y0, C, -(y1*S))`` and ``out1 = fma(y0, S, y1*C)``
    with the inner product rounded and the fused multiply-add rounded once.  The other
    columns are ``f32(acc)*(sA*sB)``.  The result is rounded to f16.
    """
    acc = gemm_i32(A_i8, B_i8).float()
    sa = scale_a.float()[:, None]
    sb = scale_b.float()[None, :]
    out = acc * (sa * sb)
    y = acc * sb
    rh = rotary_dim // 2
    seq = torch.arange(acc.shape[0]) % seqlen
    C = sa * cos_buf[seq].float()
    S = sa * sin_buf[seq].float()
    for hs in range(0, 2 * nhead * head_dim, head_dim):
        y0 = y[:, hs:hs + rh]
        y1 = y[:, hs + rh:hs + rotary_dim]
        out[:, hs:hs + rh] = fma_f32(y0, C, -(y1 * S))
        out[:, hs + rh:hs + rotary_dim] = fma_f32(y0, S, y1 * C)
    return out.to(torch.float16)


def dual_gemm_silu_ref(A_i8, Bg_i8, Bu_i8, scale_a, scale_bg, scale_bu):
    """fp32 reference of ``silu(A.Bg^T) * (A.Bu^T)``.

    Follows ``cute/ampere_dual_gemm_i8_silu.py:503-510``.
    """
    A_dq = A_i8.float() * scale_a[:, None]
    gate = A_dq @ (Bg_i8.float() * scale_bg[:, None]).T
    up = A_dq @ (Bu_i8.float() * scale_bu[:, None]).T
    return gate * torch.sigmoid(gate) * up


def dual_gemm_silu_model(A_i8, Bg_i8, Bu_i8, scale_a, scale_bg, scale_bu):
    """Model of the device epilogue on exact accumulators (kernel formula at
    ``cute/ampere_dual_gemm_i8_silu.py:426-436``): ``gate*(1/(1+exp(-gate)))*up`` -> f16.
    """
    g = gemm_i32(A_i8, Bg_i8).float() * (scale_a[:, None] * scale_bg[None, :])
    u = gemm_i32(A_i8, Bu_i8).float() * (scale_a[:, None] * scale_bu[None, :])
    sig = 1.0 / (1.0 + torch.exp(-g))
    return (g * sig * u).to(torch.float16)


# ----------------------------------------------------------------------------
# FP8 (E4M3) twins.  The reference keeps FP8 weights as B[K,N]; the device
# library takes them K-major as W[N,K] = B^T, which is what these take too.
# ----------------------------------------------------------------------------
def naive_fp8_gemm_ref(A_fp8, B_kn_fp8, scale_a, scale_b):
    """Follows ``fly/verify_fp8_gemm.py:27-40`` (bf16 result, B as [K,N])."""
    C = (A_fp8.float() * scale_a[:, None]) @ (B_kn_fp8.float() * scale_b[None, :])
    return C.to(torch.bfloat16)


def fp8_gemm_f16_ref(A_fp8, W_nk_fp8, scale_a, scale_b):
    """fp32 dequantise-then-matmul reference with W given K-major ``[N,K]``
    (same math as ``fly/verify_fp8_gemm.py:36-39``)."""
    return (A_fp8.float() * scale_a[:, None]) @ (W_nk_fp8.float() * scale_b[:, None]).T


def fp8_gemm_model(A_fp8, W_nk_fp8, scale_a, scale_b):
    """Kernel formula ``(A.B)_f32 * sA[m] * sB[n]`` (``fly/rdna_fp8_preshuffle_gemm.py:392-396``),
    accumulated in float64 so the only difference from the device is its fp32
    accumulation order."""
    acc = (A_fp8.double() @ W_nk_fp8.double().T).float()
    return acc * scale_a[:, None] * scale_b[None, :]


def fp8_rotary_ref(A_fp8, W_nk_fp8, scale_a, scale_b, sin_buf, cos_buf,
                   nhead, head_dim, rotary_dim, seqlen):
    """Follows ``fly/bench_fp8_gemm_rotary_vs_openfish.py:91-122``."""
    C = fp8_gemm_f16_ref(A_fp8, W_nk_fp8, scale_a, scale_b)
    return _rotate(C, sin_buf, cos_buf, nhead, head_dim, rotary_dim, seqlen)


def fp8_dual_silu_ref(A_fp8, Wg_nk, Wu_nk, scale_a, scale_bg, scale_bu):
    """Follows ``fly/bench_fp8_dual_gemm_silu.py:62-68``."""
    A_dq = A_fp8.float() * scale_a[:, None]
    gate = A_dq @ (Wg_nk.float() * scale_bg[:, None]).T
    up = A_dq @ (Wu_nk.float() * scale_bu[:, None]).T
    return gate * torch.sigmoid(gate) * up
