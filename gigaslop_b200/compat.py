"""Mirrors of the reference's Python kernel interface, for callers written against it.

The reference exposes each CUDA kernel as a class that is compiled and then called with tensors
(``TensorOpGemmI8`` cute/ampere_gemm_i8_quant_rmem.py:181, ``TensorOpGemmI8Rotary`` cute/ampere_gemm_i8_rotary.py:44,
``TensorOpDualGemmI8Silu`` cute/ampere_dual_gemm_i8_silu.py:36) and each RDNA kernel as a ``compile_*`` factory
returning ``launcher(out..., in..., stream[, M])`` (fly/rdna_fp8_*.py).  Here the same names wrap the B200
library; tile / atom-layout / stage arguments are accepted and ignored (tiles are fixed by the tcgen05 kernels),
tensors are torch CUDA tensors ``[rows, inner]`` (a trailing batch mode of size 1 is squeezed), weights K-major.
"""
import torch

from . import ops


def _2d(t):
    return t[..., 0] if t.dim() == 3 and t.shape[-1] == 1 else t


class _Stream:
    def __init__(self, stream):
        self.stream = stream

    def __enter__(self):
        if self.stream is not None and not isinstance(self.stream, torch.cuda.Stream):
            self.stream = torch.cuda.ExternalStream(int(self.stream))
        self.ctx = torch.cuda.stream(self.stream) if self.stream is not None else None
        if self.ctx:
            self.ctx.__enter__()

    def __exit__(self, *a):
        if self.ctx:
            self.ctx.__exit__(*a)


class TensorOpGemmI8:
    """``mC = f16((mA . mB^T) * mScaleA[m] * mScaleB[n])``; call order as the reference's ``__call__``."""

    def __init__(self, *args, **kwargs):
        self.config = (args, kwargs)

    def __call__(self, mA, mB, mC, mScaleA, mScaleB, stream=None):
        with _Stream(stream):
            ops.gemm_i8(_2d(mA), _2d(mB), _2d(mScaleA).reshape(-1), _2d(mScaleB).reshape(-1), out=_2d(mC))
        return mC


class TensorOpGemmI8Rotary:
    def __init__(self, *args, nhead=8, head_dim=64, rotary_dim=64, seqlen=1024, **kwargs):
        self.nhead, self.head_dim, self.rotary_dim, self.seqlen = nhead, head_dim, rotary_dim, seqlen

    def __call__(self, mA, mB, mC, mScaleA, mScaleB, mSin, mCos, seqlen=None, stream=None):
        with _Stream(stream):
            ops.gemm_i8_rotary(_2d(mA), _2d(mB), _2d(mScaleA).reshape(-1), _2d(mScaleB).reshape(-1), mSin, mCos,
                               self.nhead, self.head_dim, self.rotary_dim, seqlen or self.seqlen, out=_2d(mC))
        return mC


class TensorOpDualGemmI8Silu:
    def __init__(self, *args, **kwargs):
        self.config = (args, kwargs)

    def __call__(self, mA, mB_gate, mB_up, mC, mScaleA, mScaleB_gate, mScaleB_up, stream=None):
        with _Stream(stream):
            ops.dual_gemm_i8_silu(_2d(mA), _2d(mB_gate), _2d(mB_up), _2d(mScaleA).reshape(-1),
                                  _2d(mScaleB_gate).reshape(-1), _2d(mScaleB_up).reshape(-1), out=_2d(mC))
        return mC


def compile_fp8_per_token_quantize(*, K):
    """launcher(out_fp8, scale_a, inp_fp16, m, stream) -- fly/rdna_fp8_per_token_quantize.py:41-173."""
    def launcher(out_fp8, scale_a, inp, m, stream=None):
        with _Stream(stream):
            ops.fp8_quantize_per_token(inp[:m], torch_formulation=False, out=out_fp8[:m], out_scale=scale_a[:m])
    return launcher


def compile_fp8_gemm(*, M=None, N=None, K=None, **_):
    """launcher(C, A, B_nk, scale_a, scale_b, stream[, M]) -- fly/rdna_fp8_preshuffle_gemm.py:94-421 (B K-major here)."""
    def launcher(C, A, B_nk, scale_a, scale_b, stream=None, m=None):
        m = m or A.shape[0]
        with _Stream(stream):
            ops.gemm_fp8(A[:m], B_nk, scale_a[:m], scale_b, out=C[:m])
    return launcher


def compile_fp8_gemm_rotary(*, M=None, N=None, K=None, nhead=8, head_dim=64, rotary_dim=64, **_):
    """launcher(C, A, B_nk, scale_a, scale_b, sin, cos, stream, M, seqlen) -- fly/rdna_fp8_gemm_rotary.py:64-421."""
    def launcher(C, A, B_nk, scale_a, scale_b, sin, cos, stream, m, seqlen):
        with _Stream(stream):
            ops.gemm_fp8_rotary(A[:m], B_nk, scale_a[:m], scale_b, sin, cos, nhead, head_dim, rotary_dim, seqlen, out=C[:m])
    return launcher


def compile_fp8_dual_gemm_silu(*, M=None, N=None, K=None, **_):
    """launcher(C, A, Bg_nk, Bu_nk, scale_a, sbg, sbu, stream, M) -- fly/rdna_fp8_dual_gemm_silu.py:70-395."""
    def launcher(C, A, Bg, Bu, scale_a, sbg, sbu, stream, m):
        with _Stream(stream):
            ops.dual_gemm_fp8_silu(A[:m], Bg, Bu, scale_a[:m], sbg, sbu, out=C[:m])
    return launcher


def compile_fp8_down_proj(*, C=None, R=None, n_split=1, **_):
    """launcher(x_down, x, scale_x, dn_rc, scale_dn, stream, M) -- fly/rdna_fp8_factored_gemm.py:442-651."""
    def launcher(x_down, x, scale_x, dn_rc, scale_dn, stream, m):
        with _Stream(stream):
            ops.fp8_down_proj(x[:m], scale_x[:m], dn_rc, scale_dn, out=x_down[:m])
    return launcher


def compile_fp8_factored_gemm(*, C=None, R=None, N=None, **_):
    """launcher(ih, x_fp8, scale_x, dn_rc, scale_dn, up_nr, bias, stream, M) --
    fly/rdna_fp8_factored_gemm.py:86-435 (argument order of fly/bench_factored_gemm.py:46-50); ``dn`` ``[R, C]``
    and ``up`` ``[N, R]`` K-major instead of the RDNA pre-shuffles."""
    def launcher(ih, x, scale_x, dn_rc, scale_dn, up_nr, bias, stream, m):
        with _Stream(stream):
            ops.fp8_factored_gemm(x[:m], scale_x[:m], dn_rc, scale_dn, up_nr, bias, out=ih[:m])
    return launcher


def compile_fp8_factored_lstm(*, B=None, H=None, K_hh=None, R=None, **_):
    """launcher(h_fp8, c, hh_down, up_hh_nk, bias_hh, x_down, up_ih_nk, bias_ih, stream, B) --
    fly/rdna_fp8_factored_lstm.py:88-351."""
    def launcher(h_fp8, c, hh_down, up_hh, bias_hh, x_down, up_ih, bias_ih, stream, b):
        with _Stream(stream):
            ops.factored_lstm_step(h_fp8[:b], c[:b], hh_down[:b], up_hh, bias_hh, x_down[:b], up_ih, bias_ih)
    return launcher
