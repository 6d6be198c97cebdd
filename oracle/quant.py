"""Oracle: activation / weight quantisers (CPU, PyTorch).  Test infrastructure only.

Restates the reference's host-side quantisers.  All arithmetic is fp32 on CPU
tensors, in the same operation order as the reference, because the order
(multiply by ``127/amax`` versus divide by ``amax/127``) changes individual
int8 values and scale ulps.
"""
import numpy as np
import torch

FP8_MAX = 448.0


def quantize_tensor(t, dim=-1):
    """Symmetric per-row absmax int8 quantiser (the canonical INT8 quantiser).

    Follows ``cute/bench_quant_i8.py:15-31`` (identical copies at
    ``cute/test_gemm_i8_rotary_vs_openfish.py:35-40``,
    ``cute/bench_gemm_i8_rotary.py:15-20``, ``cute/bench_dual_gemm_i8_silu.py:15-20``):
    amax clamped to 1e-8, ``qs = 127/amax``, ``q = round_half_even(t*qs)``
    clamped to +-127, dequant scale ``= 1/qs``.  ``t`` must be fp32.  Note that
    PyTorch evaluates ``127 / tensor`` (Python scalar numerator) as
    ``tensor.reciprocal() * 127`` -- two roundings, not one IEEE division -- and the
    device kernel reproduces exactly that.
    """
    qm = 127
    fr = t.abs().amax(dim=dim).clamp_min(1e-8)
    qs = qm / fr
    ti = (t * qs.unsqueeze(dim)).round().clamp(-qm, qm).to(torch.int8)
    return ti, qs.to(torch.float32).reciprocal()


def quantize_per_row_cpp(x):
    """The C++ consumer's quantiser: as above but rounds half away from zero.

    Follows ``cute/main.cpp:27-56`` / ``cute/main_rotary.cpp:61-74``
    (``std::round``).  Used only to rebuild those programs' host inputs.
    """
    x = x.float()
    amax = x.abs().amax(dim=-1).clamp_min(1e-8)
    qs = 127.0 / amax
    s = x * qs[:, None]
    r = torch.sign(s) * torch.floor(s.abs() + 0.5)
    return r.clamp(-127, 127).to(torch.int8), (1.0 / qs)


def fp8_quantize_per_token(x_f32):
    """Per-token E4M3 quantiser, torch formulation (divide by ``amax/448``).

    Follows ``fly/rdna_fp8_preshuffle_gemm.py:57-70`` (duplicates at
    ``fly/rdna_fp8_gemm_rotary.py:42-48``, ``fly/rdna_fp8_factored_gemm.py:64-70``).
    Returns (float8_e4m3fn [M,K], fp32 scale [M]).
    """
    amax = x_f32.abs().amax(dim=-1, keepdim=True).clamp(min=1e-12)
    scale = amax / FP8_MAX
    x_scaled = (x_f32 / scale).clamp(-FP8_MAX, FP8_MAX)
    return x_scaled.to(torch.float8_e4m3fn), scale.squeeze(-1)


def fp8_quantize_per_token_kernel(x_f32):
    """Per-token E4M3 quantiser, kernel formulation (multiply by ``448/amax``).

    Follows the device code at ``fly/rdna_fp8_per_token_quantize.py:127-148``:
    ``inv = 448/amax``, ``scale = amax/448``, elements converted from ``x*inv``
    with round-to-nearest-even and saturation to +-448.
    """
    amax = x_f32.abs().amax(dim=-1, keepdim=True).clamp(min=1e-12)
    inv = torch.full_like(amax, FP8_MAX) / amax          # a true IEEE division, as the device code does
    scale = amax / FP8_MAX
    q = (x_f32 * inv).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale.squeeze(-1)


def fp8_quantize_per_channel(x_f32):
    """Per-column E4M3 weight quantiser for ``B[K,N]``.

    Follows ``fly/rdna_fp8_preshuffle_gemm.py:73-86``.
    """
    amax = x_f32.abs().amax(dim=0).clamp(min=1e-12)
    scale = amax / FP8_MAX
    x_scaled = (x_f32 / scale.unsqueeze(0)).clamp(-FP8_MAX, FP8_MAX)
    return x_scaled.to(torch.float8_e4m3fn), scale


def fp8_quantize_scalar(x_f32):
    """Single-scale E4M3 quantiser.  Follows ``fly/rdna_fp8_factored_gemm.py:73-79``."""
    amax = x_f32.abs().amax().clamp(min=1e-12)
    scale = (amax / FP8_MAX).reshape(1)
    q = (x_f32 / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale


# --------------------------------------------------------------------------
# Software E4M3 codec (numpy).  Independent restatement of the OCP FP8 E4M3
# ("fn": no infinities, S.1111.111 is NaN, max finite 448) used to cross-check
# torch's cast and to decode raw device bytes without going through torch.
# --------------------------------------------------------------------------
def e4m3_decode(b):
    """uint8 array -> float32 array (OCP E4M3FN)."""
    b = np.asarray(b, dtype=np.uint8).astype(np.int32)
    sign = np.where(b & 0x80, -1.0, 1.0)
    e = (b >> 3) & 0xF
    m = b & 0x7
    val = np.where(e == 0, m * 2.0 ** -9, (8 + m) * 2.0 ** (e.astype(np.float64) - 10))
    val = np.where((e == 15) & (m == 7), np.nan, val)
    return (sign * val).astype(np.float32)


def e4m3_encode(x):
    """float32 array -> uint8 E4M3FN, round-to-nearest-even, saturating to +-448.

    This is the behaviour of a saturating-finite hardware convert; NaN maps to 0x7f.
    """
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x).astype(np.float64)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    a = np.minimum(a, 448.0)
    # exponent of the containing binade, clamped to the subnormal binade
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.clip(e, -6, 8)
    step = 2.0 ** (e - 3)                       # spacing inside the binade
    q = np.rint(a / step)                       # numpy rint = half to even
    v = q * step                                # may carry into next binade
    v = np.minimum(v, 448.0)
    # re-derive fields from the rounded value
    with np.errstate(divide="ignore"):
        e2 = np.floor(np.log2(np.where(v > 0, v, 1.0)))
    sub = v < 2.0 ** -6
    e2 = np.clip(e2, -6, 8)
    mant = np.where(sub, v / 2.0 ** -9, v / 2.0 ** (e2 - 3) - 8)
    expf = np.where(sub, 0, e2 + 7)
    out = (expf.astype(np.uint8) << 3) | mant.astype(np.uint8)
    out = np.where(np.isnan(x), 0x7F, out | sign)
    return out.astype(np.uint8)
