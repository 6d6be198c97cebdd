"""PyTorch-facing host functions over the C ABI.  torch supplies device memory
and streams; every byte of compute happens in libgigaslop_b200.so.

Function names and argument meaning follow the reference's host helpers
(``quantize_tensor``, ``fp8_quantize_per_token``) and kernels.
"""
import functools

import torch

from . import _lib
from ._lib import check, lib


def _stream(t=None):
    """Current stream of ``t``'s device (of the current device without ``t``: inside an ``@_on_device`` function
    that is the tensors' device)."""
    return torch.cuda.current_stream(t.device if t is not None else None).cuda_stream


def same_device(*ts):
    """The one device all given tensors live on.  CPU tensors raise (there is no CPU path); tensors spread over
    several devices raise (the library launches on one device and would reach the others through peer pointers,
    with the wrong device's kernel attributes, SM count and static scratch)."""
    dev = None
    for t in ts:
        if t is None:
            continue
        if t.device.type != "cuda":
            raise RuntimeError("gigaslop_b200 operates on CUDA tensors only (no CPU fallback)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"all tensors of one call must live on one device (got {dev} and {t.device})")
    return dev


_need_cuda = same_device


def _on_device(fn):
    """Run ``fn`` with the device of its tensor arguments current: the C side keys its per-device state on the
    current device, and ``_stream()`` then returns that device's current stream."""
    @functools.wraps(fn)
    def wrapped(*args, **kwargs):
        dev = same_device(*[a for a in args if isinstance(a, torch.Tensor)],
                          *[a for a in kwargs.values() if isinstance(a, torch.Tensor)])
        if dev is None or dev.index == torch.cuda.current_device():      # the common case costs no context switch
            return fn(*args, **kwargs)
        with torch.cuda.device(dev):
            return fn(*args, **kwargs)
    return wrapped


def _rowmajor(t, name):
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with unit inner stride")
    return t


def _dt(t):
    if t.dtype == torch.float16:
        return _lib.F16
    if t.dtype == torch.float32:
        return _lib.F32
    raise TypeError("activations must be float16 or float32")


@_on_device
def quantize_tensor(t, dim=-1, out=None, out_scale=None):
    """Per-row symmetric absmax INT8 quantiser; same contract as the reference's
    ``quantize_tensor`` (cute/bench_quant_i8.py:15-31): returns (int8 [M,K], fp32 dequant scale [M])."""
    if dim not in (-1, t.dim() - 1):
        raise ValueError("only per-row (last-dim) quantisation is on the hot path")
    _need_cuda(t)
    x = _rowmajor(t, "t")
    M, K = x.shape
    q = out if out is not None else torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = out_scale if out_scale is not None else torch.empty((M,), dtype=torch.float32, device=x.device)
    check(lib().gsb200_ptq_int8(x.data_ptr(), _dt(x), x.stride(0), q.data_ptr(), q.stride(0), s.data_ptr(),
                                M, K, _stream()), "quantize_tensor")
    return q, s


@_on_device
def fp8_quantize_per_token(x, torch_formulation=True, out=None, out_scale=None):
    """Per-row E4M3 quantiser (fly/rdna_fp8_preshuffle_gemm.py:57-70); ``torch_formulation=False``
    selects the device-kernel arithmetic of fly/rdna_fp8_per_token_quantize.py."""
    _need_cuda(x)
    x = _rowmajor(x, "x")
    M, K = x.shape
    q = out if out is not None else torch.empty((M, K), dtype=torch.float8_e4m3fn, device=x.device)
    s = out_scale if out_scale is not None else torch.empty((M,), dtype=torch.float32, device=x.device)
    check(lib().gsb200_ptq_fp8(x.data_ptr(), _dt(x), x.stride(0), q.data_ptr(), q.stride(0), s.data_ptr(),
                               M, K, 1 if torch_formulation else 0, _stream()), "fp8_quantize_per_token")
    return q, s


def _check_ab(A, B, dtypes):
    _need_cuda(A, B)
    _rowmajor(A, "A"); _rowmajor(B, "B")
    if A.dtype not in dtypes or B.dtype not in dtypes:
        raise TypeError(f"operands must be one of {dtypes}")
    if A.shape[1] != B.shape[1]:
        raise ValueError("A is [M,K], B is [N,K]: K mismatch")
    return A.shape[0], B.shape[0], A.shape[1]


_I8 = (torch.int8,)
_F8 = (torch.float8_e4m3fn, torch.uint8)


@_on_device
def gemm_i8_i32(A, B, out=None):
    """Exact int32 ``A[M,K] . B[N,K]^T`` (cute/ampere_gemm_i8.py TensorOpGemmI8, int32 output)."""
    M, N, K = _check_ab(A, B, _I8)
    C = out if out is not None else torch.empty((M, N), dtype=torch.int32, device=A.device)
    check(lib().gsb200_gemm_i8_i32(A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), C.data_ptr(), C.stride(0),
                                   M, N, K, _stream()), "gemm_i8_i32")
    return C


def _gemm_f16(fn, name, A, B, scale_a, scale_b, out, flags, dtypes):
    M, N, K = _check_ab(A, B, dtypes)
    _need_cuda(scale_a, scale_b)
    C = out if out is not None else torch.empty((M, N), dtype=torch.float16, device=A.device)
    check(fn(A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), C.data_ptr(), C.stride(0),
             scale_a.data_ptr(), scale_b.data_ptr(), M, N, K, flags, _stream()), name)
    return C


@_on_device
def gemm_i8(A, B, scale_a, scale_b, out=None, flags=0):
    """W8A8 GEMM with per-token x per-channel dequant to fp16 (cute/ampere_gemm_i8_quant_rmem.py)."""
    return _gemm_f16(lib().gsb200_gemm_i8_f16, "gemm_i8", A, B, scale_a, scale_b, out, flags, _I8)


@_on_device
def gemm_fp8(A, B, scale_a, scale_b, out=None, flags=0):
    """FP8 GEMM, ``B`` K-major ``[N,K]`` (fly/rdna_fp8_preshuffle_gemm.py compile_fp8_gemm)."""
    return _gemm_f16(lib().gsb200_gemm_fp8_f16, "gemm_fp8", A, B, scale_a, scale_b, out, flags, _F8)


def _rotary(fn, name, A, B, scale_a, scale_b, sin_buf, cos_buf, nhead, head_dim, rotary_dim, seqlen,
            row_offset, out, flags, dtypes):
    M, N, K = _check_ab(A, B, dtypes)
    _need_cuda(scale_a, scale_b, sin_buf, cos_buf)
    if sin_buf.dtype != torch.float32 or not sin_buf.is_contiguous() or not cos_buf.is_contiguous():
        raise ValueError("sin/cos must be contiguous float32 [seqlen, rotary_dim/2]")
    if sin_buf.shape[0] < seqlen or sin_buf.shape[1] != rotary_dim // 2:
        raise ValueError("sin/cos table smaller than seqlen")
    C = out if out is not None else torch.empty((M, N), dtype=torch.float16, device=A.device)
    check(fn(A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), C.data_ptr(), C.stride(0),
             scale_a.data_ptr(), scale_b.data_ptr(), sin_buf.data_ptr(), cos_buf.data_ptr(),
             M, N, K, nhead, head_dim, rotary_dim, seqlen, row_offset, flags, _stream()), name)
    return C


@_on_device
def gemm_i8_rotary(A, B, scale_a, scale_b, sin_buf, cos_buf, nhead, head_dim, rotary_dim, seqlen,
                   row_offset=0, out=None, flags=0):
    """QKV GEMM + rotary epilogue (cute/ampere_gemm_i8_rotary.py TensorOpGemmI8Rotary)."""
    return _rotary(lib().gsb200_gemm_i8_rotary_f16, "gemm_i8_rotary", A, B, scale_a, scale_b, sin_buf, cos_buf,
                   nhead, head_dim, rotary_dim, seqlen, row_offset, out, flags, _I8)


@_on_device
def quantize_gemm_i8_rotary(x, B, scale_b, sin_buf, cos_buf, nhead, head_dim, rotary_dim, seqlen,
                            row_offset=0, out=None, out_scale=None, flags=0):
    """``gemm_i8_rotary(*quantize_tensor(x), ...)`` in one launch: fp16 ``x`` [M, K] in, the int8 operand is made on
    chip.  Same bytes as the two calls.  ``out_scale`` (optional, [M] fp32) receives the token scales."""
    _need_cuda(x, B, scale_b, sin_buf, cos_buf)
    if x.dtype != torch.float16 or B.dtype != torch.int8 or x.dim() != 2 or B.dim() != 2 or x.shape[1] != B.shape[1]:
        raise ValueError("x must be fp16 [M, K] and B int8 [N, K]")
    if x.stride(1) != 1 or B.stride(1) != 1:
        raise ValueError("rows must be contiguous")
    if sin_buf.dtype != torch.float32 or not sin_buf.is_contiguous() or not cos_buf.is_contiguous():
        raise ValueError("sin/cos must be contiguous float32 [seqlen, rotary_dim/2]")
    if sin_buf.shape[0] < seqlen or sin_buf.shape[1] != rotary_dim // 2:
        raise ValueError("sin/cos table smaller than seqlen")
    M, K = x.shape
    N = B.shape[0]
    C = out if out is not None else torch.empty((M, N), dtype=torch.float16, device=x.device)
    if out_scale is not None and (out_scale.dtype != torch.float32 or out_scale.numel() < M or not out_scale.is_cuda):
        raise ValueError("out_scale must be a CUDA float32 tensor of at least M elements")
    check(lib().gsb200_ptq_gemm_i8_rotary_f16(
        x.data_ptr(), x.stride(0), B.data_ptr(), B.stride(0), C.data_ptr(), C.stride(0),
        out_scale.data_ptr() if out_scale is not None else None, scale_b.data_ptr(), sin_buf.data_ptr(),
        cos_buf.data_ptr(), M, N, K, nhead, head_dim, rotary_dim, seqlen, row_offset, flags, _stream()),
        "quantize_gemm_i8_rotary")
    return C


@_on_device
def gemm_fp8_rotary(A, B, scale_a, scale_b, sin_buf, cos_buf, nhead, head_dim, rotary_dim, seqlen,
                    row_offset=0, out=None, flags=0):
    """FP8 QKV GEMM + rotary (fly/rdna_fp8_gemm_rotary.py compile_fp8_gemm_rotary)."""
    return _rotary(lib().gsb200_gemm_fp8_rotary_f16, "gemm_fp8_rotary", A, B, scale_a, scale_b, sin_buf, cos_buf,
                   nhead, head_dim, rotary_dim, seqlen, row_offset, out, flags, _F8)


def _dual(fn, name, A, Bg, Bu, scale_a, sbg, sbu, out, flags, dtypes):
    M, N, K = _check_ab(A, Bg, dtypes)
    _check_ab(A, Bu, dtypes)
    if Bu.shape != Bg.shape or Bu.stride(0) != Bg.stride(0):
        raise ValueError("gate and up weights must share shape and row stride")
    _need_cuda(scale_a, sbg, sbu)
    C = out if out is not None else torch.empty((M, N), dtype=torch.float16, device=A.device)
    check(fn(A.data_ptr(), A.stride(0), Bg.data_ptr(), Bu.data_ptr(), Bg.stride(0), C.data_ptr(), C.stride(0),
             scale_a.data_ptr(), sbg.data_ptr(), sbu.data_ptr(), M, N, K, flags, _stream()), name)
    return C


@_on_device
def dual_gemm_i8_silu(A, B_gate, B_up, scale_a, scale_b_gate, scale_b_up, out=None, flags=0):
    """``silu(A.Bg^T) * (A.Bu^T)`` (cute/ampere_dual_gemm_i8_silu.py TensorOpDualGemmI8Silu)."""
    return _dual(lib().gsb200_dual_gemm_i8_silu_f16, "dual_gemm_i8_silu", A, B_gate, B_up, scale_a,
                 scale_b_gate, scale_b_up, out, flags, _I8)


@_on_device
def dual_gemm_fp8_silu(A, B_gate, B_up, scale_a, scale_b_gate, scale_b_up, out=None, flags=0):
    """FP8 SwiGLU dual GEMM (fly/rdna_fp8_dual_gemm_silu.py compile_fp8_dual_gemm_silu)."""
    return _dual(lib().gsb200_dual_gemm_fp8_silu_f16, "dual_gemm_fp8_silu", A, B_gate, B_up, scale_a,
                 scale_b_gate, scale_b_up, out, flags, _F8)


@_on_device
def mxfp8_quantize(x, out=None, out_scale=None):
    """Activations [M,K] fp16/fp32 -> (float8_e4m3fn [M,K], uint8 E8M0 scales [M,K/32]); one scale per 32 elements."""
    _need_cuda(x)
    x = _rowmajor(x, "x")
    M, K = x.shape
    q = out if out is not None else torch.empty((M, K), dtype=torch.float8_e4m3fn, device=x.device)
    s = out_scale if out_scale is not None else torch.empty((M, K // 32), dtype=torch.uint8, device=x.device)
    check(lib().gsb200_ptq_mxfp8(x.data_ptr(), _dt(x), x.stride(0), q.data_ptr(), q.stride(0), s.data_ptr(),
                                 s.stride(0), M, K, _stream()), "mxfp8_quantize")
    return q, s


@_on_device
def dual_gemm_fp8_silu_mxfp8(A, B_gate, B_up, scale_a, scale_b_gate, scale_b_up, out=None, out_scale=None, flags=0):
    """FP8 SwiGLU dual GEMM emitting MXFP8 (elements + E8M0 scale per 32 output columns); the interface of
    fp8_dual_silu_mxfp8_wrapper (fly/export_fp8_dual_gemm_silu_mxfp8.py:206-236)."""
    M, N, K = _check_ab(A, B_gate, _F8)
    _check_ab(A, B_up, _F8)
    _need_cuda(scale_a, scale_b_gate, scale_b_up)
    q = out if out is not None else torch.empty((M, N), dtype=torch.float8_e4m3fn, device=A.device)
    s = out_scale if out_scale is not None else torch.empty((M, N // 32), dtype=torch.uint8, device=A.device)
    check(lib().gsb200_dual_gemm_fp8_silu_mxfp8(
        A.data_ptr(), A.stride(0), B_gate.data_ptr(), B_up.data_ptr(), B_gate.stride(0), q.data_ptr(), q.stride(0),
        s.data_ptr(), s.stride(0), scale_a.data_ptr(), scale_b_gate.data_ptr(), scale_b_up.data_ptr(), M, N, K, flags,
        _stream()), "dual_gemm_fp8_silu_mxfp8")
    return q, s


@_on_device
def gemm_f16(A, B, scale_a=None, scale_b=None, out=None, flags=0):
    """``(A_f16 . B_f16^T) * sA * sB`` -> fp16, scales optional (compile_f16_down_proj,
    fly/rdna_fp8_factored_gemm.py:660-843, is this with no scales and B = dn ``[R, C]``)."""
    M, N, K = _check_ab(A, B, (torch.float16,))
    C = out if out is not None else torch.empty((M, N), dtype=torch.float16, device=A.device)
    check(lib().gsb200_gemm_f16_f16(A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), C.data_ptr(), C.stride(0),
                                    scale_a.data_ptr() if scale_a is not None else None,
                                    scale_b.data_ptr() if scale_b is not None else None, M, N, K, flags, _stream()),
          "gemm_f16")
    return C


@_on_device
def fp8_down_proj(x_fp8, scale_x, dn_fp8_rc, scale_dn, out=None):
    """``x_down_f16[M,R] = (x_fp8 . dn_fp8^T) * sx[m] * s_dn`` with a single scalar weight scale
    (compile_fp8_down_proj, fly/rdna_fp8_factored_gemm.py:442-651); ``dn`` K-major ``[R, C]``."""
    return gemm_fp8(x_fp8, dn_fp8_rc, scale_x, scale_dn, out=out, flags=_lib.FLAG_SCALAR_SCALE_B)


@_on_device
def fp8_factored_gemm(x_fp8, scale_x, dn_fp8_rc, scale_dn, up_f16_nr, bias, out=None):
    """Hoisted low-rank input projection ``ih = f16(f16((x . dn^T) * sx * s_dn) . up^T + bias)`` in one call
    (compile_fp8_factored_gemm, fly/rdna_fp8_factored_gemm.py:86-435).  ``dn`` ``[R, C]`` E4M3 and ``up``
    ``[N, R]`` fp16, both K-major; the intermediate lives inside ``out`` between the two launches."""
    _need_cuda(x_fp8, scale_x, dn_fp8_rc, scale_dn, up_f16_nr, bias)
    _rowmajor(x_fp8, "x"); _rowmajor(dn_fp8_rc, "dn"); _rowmajor(up_f16_nr, "up")
    if x_fp8.dtype != torch.float8_e4m3fn or dn_fp8_rc.dtype != torch.float8_e4m3fn or up_f16_nr.dtype != torch.float16:
        raise TypeError("x and dn must be float8_e4m3fn, up float16")
    M, C = x_fp8.shape
    R, C2 = dn_fp8_rc.shape
    N, R2 = up_f16_nr.shape
    if C2 != C or R2 != R or bias.numel() != N or scale_x.numel() != M:
        raise ValueError("shape mismatch")
    ih = out if out is not None else torch.empty((M, N), dtype=torch.float16, device=x_fp8.device)
    check(lib().gsb200_fac_gemm_fp8_f16(x_fp8.data_ptr(), x_fp8.stride(0), scale_x.data_ptr(), dn_fp8_rc.data_ptr(),
                                        dn_fp8_rc.stride(0), scale_dn.data_ptr(), up_f16_nr.data_ptr(),
                                        up_f16_nr.stride(0), bias.data_ptr(), ih.data_ptr(), ih.stride(0), M, C, R, N,
                                        _stream()), "fp8_factored_gemm")
    return ih


@_on_device
def factored_lstm_step(h_fp8_out, c_inout, hh_down, up_hh, bias_hh, x_down, up_ih, bias_ih):
    """One step of the low-rank hard-gate LSTM cell; argument order of fp8_factored_lstm_wrapper
    (fly/export_fp8_factored_lstm.py:158-182).  ``up_hh`` ``[4H, K_hh]`` and ``up_ih`` ``[4H, R]`` fp16 K-major."""
    _need_cuda(h_fp8_out, c_inout, hh_down, up_hh, x_down, up_ih)
    B, K_hh = hh_down.shape
    H = up_hh.shape[0] // 4
    R = x_down.shape[1]
    for t in (hh_down, up_hh, x_down, up_ih, c_inout, h_fp8_out):
        if not t.is_contiguous():
            raise ValueError("factored_lstm_step takes contiguous tensors")
    check(lib().gsb200_factored_lstm_step(h_fp8_out.data_ptr(), c_inout.data_ptr(), hh_down.data_ptr(), up_hh.data_ptr(),
                                          bias_hh.data_ptr() if bias_hh is not None else None, x_down.data_ptr(),
                                          up_ih.data_ptr(), bias_ih.data_ptr() if bias_ih is not None else None,
                                          B, H, K_hh, R, _stream()), "factored_lstm_step")
    return h_fp8_out, c_inout


@_on_device
def mx_scales_to_tiled(scales, K):
    """Row-major E8M0 scales ``[rows, K/32]`` -> the 128 x 4 tile order the block-scaled GEMMs take."""
    _need_cuda(scales)
    rows = scales.shape[0]
    out = torch.empty(int(lib().gsb200_mx_tiled_scale_bytes(rows, K)), dtype=torch.uint8, device=scales.device)
    check(lib().gsb200_mx_scales_to_tiled(scales.data_ptr(), scales.stride(0), rows, K, out.data_ptr(), _stream()),
          "mx_scales_to_tiled")
    return out


@_on_device
def gemm_mxfp8(A, sfa_tiled, B, sfb_tiled, out=None):
    """Block-scaled MXFP8 GEMM ``A[M,K] . B[N,K]^T`` (E8M0 scale per 32 K elements on both operands) -> fp16."""
    M, N, K = _check_ab(A, B, _F8)
    C = out if out is not None else torch.empty((M, N), dtype=torch.float16, device=A.device)
    check(lib().gsb200_gemm_mxfp8_f16(A.data_ptr(), A.stride(0), sfa_tiled.data_ptr(), B.data_ptr(), B.stride(0),
                                      sfb_tiled.data_ptr(), C.data_ptr(), C.stride(0), M, N, K, _stream()), "gemm_mxfp8")
    return C


@_on_device
def dual_gemm_mxfp8_silu(A, sfa_tiled, B_gate, B_up, sfb_gate_tiled, sfb_up_tiled, out=None):
    """Block-scaled MXFP8 SwiGLU dual GEMM ``silu(A.Bg^T) * (A.Bu^T)`` -> fp16."""
    M, N, K = _check_ab(A, B_gate, _F8)
    _check_ab(A, B_up, _F8)
    C = out if out is not None else torch.empty((M, N), dtype=torch.float16, device=A.device)
    check(lib().gsb200_dual_gemm_mxfp8_silu_f16(A.data_ptr(), A.stride(0), sfa_tiled.data_ptr(), B_gate.data_ptr(),
                                                B_up.data_ptr(), B_gate.stride(0), sfb_gate_tiled.data_ptr(),
                                                sfb_up_tiled.data_ptr(), C.data_ptr(), C.stride(0), M, N, K, _stream()),
          "dual_gemm_mxfp8_silu")
    return C
