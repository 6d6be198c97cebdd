"""GPU parity of the GEMM kernel variants: eight or twelve epilogue warps, one CTA or a CTA pair per tile.

Which variant runs is normally chosen by shape; gsb200_set_gemm_variant forces one, so every variant is held to the CPU oracle on shapes with ragged row and column counts, an odd number of
row blocks (the second CTA of the last pair has no rows), every schedule (weight-stationary, activation-stationary,
streaming) and both operand kinds.  All variants must give the same bytes."""
import pytest
import torch

import oracle
from util import assert_bitexact, f16_equal_up_to_signed_zero, need_lib, rand_i8, rand_scales

pytestmark = pytest.mark.gpu

VARIANTS = [(8, 0), (8, 1), (12, 0), (12, 1)]


@pytest.fixture
def force():
    """force(ew, pair) selects a variant; the by-shape choice is restored afterwards."""
    g = need_lib()
    def set_variant(ew, pair):
        assert g.lib().gsb200_set_gemm_variant(ew, pair) == 0
    yield set_variant
    g.lib().gsb200_set_gemm_variant(-1, -1)


@pytest.mark.parametrize("ew,pair", VARIANTS)
@pytest.mark.parametrize("M,N,K", [(128, 256, 256), (129, 520, 512), (1000, 1536, 384), (4096 + 130, 512, 2048), (70000, 512, 256)])
def test_dequant_variants(force, ew, pair, M, N, K):
    g = need_lib()
    force(ew, pair)
    gen = torch.Generator().manual_seed(77 + M + N + K)
    A, B = rand_i8(gen, M, K), rand_i8(gen, N, K)
    sa, sb = rand_scales(gen, M, 5e-3, 5e-2), rand_scales(gen, N)
    c = g.gemm_i8(A.cuda(), B.cuda(), sa.cuda(), sb.cuda())
    assert g.device_status()[0] == 0
    assert f16_equal_up_to_signed_zero(c, oracle.gemm_dequant_exact(A, B, sa, sb)) == 0


@pytest.mark.parametrize("ew,pair", VARIANTS)
@pytest.mark.parametrize("M,seqlen,row_offset,K,nhead", [(256, 333, 0, 512, 8), (1000, 2048, 1536, 512, 8), (20000 + 128, 2048, 0, 512, 8),
                                                         (700, 77, 3, 640, 3), (2500, 100, 0, 256, 6)])
def test_rotary_variants(force, ew, pair, M, seqlen, row_offset, K, nhead):
    g = need_lib()
    force(ew, pair)
    head_dim = rotary_dim = 64
    N = 3 * nhead * head_dim
    gen = torch.Generator().manual_seed(3000 + M + seqlen)
    A, sa = oracle.quantize_tensor(torch.randn(M, K, generator=gen))
    B, sb = rand_i8(gen, N, K), rand_scales(gen, N)
    sn, cs = oracle.rope_tables(max(seqlen, 16), rotary_dim // 2, head_dim)
    c = g.gemm_i8_rotary(A.cuda(), B.cuda(), sa.cuda(), sb.cuda(), sn.cuda(), cs.cuda(), nhead, head_dim, rotary_dim, seqlen,
                         row_offset=row_offset)
    assert g.device_status()[0] == 0
    Ap = torch.cat([torch.zeros(row_offset, K, dtype=torch.int8), A])
    sap = torch.cat([torch.ones(row_offset), sa])
    exact = oracle.rotary_exact(Ap, B, sap, sb, sn, cs, nhead, head_dim, rotary_dim, seqlen)[row_offset:]
    assert f16_equal_up_to_signed_zero(c, exact) == 0


@pytest.mark.parametrize("ew,pair", VARIANTS)
@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (300, 2048, 512), (65, 136, 512), (9000 + 128, 2048, 512), (2000, 512, 1024)])
def test_dual_silu_variants_agree(force, ew, pair, M, N, K):
    """SwiGLU: every variant against the default kernel's bytes at a size below the variants' threshold (the default
    there is the eight-warp single-CTA kernel, which the oracle tests of the INT8 file cover)."""
    g = need_lib()
    gen = torch.Generator().manual_seed(4000 + M + N + K)
    A, sa = oracle.quantize_tensor(torch.randn(M, K, generator=gen))
    Wg, Wu = rand_i8(gen, N, K), rand_i8(gen, N, K)
    sg, su = rand_scales(gen, N), rand_scales(gen, N)
    args = (A.cuda(), Wg.cuda(), Wu.cuda(), sa.cuda(), sg.cuda(), su.cuda())
    force(8, 0)
    base = g.dual_gemm_i8_silu(*args)
    force(ew, pair)
    got = g.dual_gemm_i8_silu(*args)
    assert g.device_status()[0] == 0
    assert_bitexact(got, base, f"SwiGLU, {ew} epilogue warps, pair={pair}")


@pytest.mark.parametrize("ew,pair", VARIANTS)
def test_fp8_variants_agree(force, ew, pair):
    g = need_lib()
    from gigaslop_b200 import ops
    gen = torch.Generator().manual_seed(5)
    M, N, K = 3000 + 128, 1536, 512
    x8, sx = ops.fp8_quantize_per_token(torch.randn(M, K, generator=gen).half().cuda())
    W = (torch.randn(N, K, generator=gen) * 50).to(torch.float8_e4m3fn).cuda()
    sw = rand_scales(gen, N).cuda()
    sn, cs = (t.cuda() for t in oracle.rope_tables(2048, 32, 64))
    outs = []
    for e, p in ((8, 0), (ew, pair)):
        force(e, p)
        outs.append((ops.gemm_fp8(x8, W, sx, sw), ops.gemm_fp8_rotary(x8, W, sx, sw, sn, cs, 8, 64, 64, 2048),
                     ops.dual_gemm_fp8_silu(x8, W[:768], W[768:], sx, sw[:768], sw[768:])))
    assert g.device_status()[0] == 0
    for a, b, what in zip(outs[0], outs[1], ("dequant", "rotary", "SwiGLU")):
        assert_bitexact(b, a, f"FP8 {what}, {ew} epilogue warps, pair={pair}")


def test_variant_setter_rejects_other_values():
    g = need_lib()
    assert g.lib().gsb200_set_gemm_variant(16, 0) != 0
    assert g.lib().gsb200_set_gemm_variant(8, 2) != 0
    assert g.lib().gsb200_set_gemm_variant(-1, -1) == 0
