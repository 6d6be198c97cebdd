"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch


def need_lib():
    import gigaslop_b200
    gigaslop_b200.lib()
    return gigaslop_b200


def close(got, ref, atol, rtol):
    """Element passes if abs err <= atol OR rel err <= rtol (the reference's own gate,
    cute/main_rotary.cpp:194,212).  Returns (ok, max_abs, n_bad)."""
    got = got.float().cpu()
    ref = ref.float().cpu()
    err = (got - ref).abs()
    bad = (err > atol) & (err > rtol * ref.abs())
    return (not bool(bad.any())), float(err.max()), int(bad.sum())


def assert_close(got, ref, atol, rtol, what=""):
    ok, mx, nbad = close(got, ref, atol, rtol)
    assert ok, f"{what}: {nbad} elements outside atol={atol} / rtol={rtol} (max abs err {mx})"


def assert_bitexact(got, ref, what=""):
    g = got.cpu().contiguous()
    r = ref.cpu().contiguous()
    assert g.shape == r.shape and g.dtype == r.dtype, f"{what}: {g.shape}/{g.dtype} vs {r.shape}/{r.dtype}"
    if g.dtype in (torch.float16, torch.bfloat16):
        g, r = g.view(torch.int16), r.view(torch.int16)
    elif g.dtype == torch.float32:
        g, r = g.view(torch.int32), r.view(torch.int32)
    elif g.dtype == torch.float8_e4m3fn:
        g, r = g.view(torch.uint8), r.view(torch.uint8)
    n = int((g != r).sum())
    assert n == 0, f"{what}: {n} of {g.numel()} elements differ bitwise"


def f16_equal_up_to_signed_zero(got, ref):
    g = got.cpu().view(torch.int16)
    r = ref.cpu().view(torch.int16)
    diff = g != r
    both_zero = ((g & 0x7FFF) == 0) & ((r & 0x7FFF) == 0)
    return int((diff & ~both_zero).sum())


def rand_i8(gen, *shape):
    return torch.randint(-127, 128, shape, generator=gen, dtype=torch.int8)


def rand_scales(gen, n, lo=1e-3, hi=1e-2):
    return lo + (hi - lo) * torch.rand(n, generator=gen)


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def rotary_rows(fn, A_rows, sa_rows, B, sb, sn, cs, nhead, head_dim, rotary_dim, seqlen, first_pos):
    """Oracle rotary GEMM (``fn`` = oracle.rotary_exact / rotary_ref / fp8_rotary_ref) for a slice of rows whose first
    row sits at sequence position ``first_pos``: the oracle takes the angle row from the row index, so the slice is
    prefixed with ``first_pos % seqlen`` zero rows that are dropped again."""
    pad = int(first_pos) % int(seqlen)
    Ap = torch.cat([torch.zeros(pad, A_rows.shape[1], dtype=A_rows.dtype), A_rows])
    sap = torch.cat([torch.ones(pad), sa_rows])
    return fn(Ap, B, sap, sb, sn, cs, nhead, head_dim, rotary_dim, seqlen)[pad:]


SAMPLE_SLICES_64K = [(0, 256), (32768 - 64, 32768 + 64), (65536 - 256, 65536), (12345, 12345 + 77)]
