"""GPU checks of the MXFP8 pieces (parity unpinned: the rule is this library's, see oracle/mx.py).
The activation quantiser is compared bit for bit with the CPU statement of the rule; the fused
SwiGLU->MXFP8 epilogue is held to the error bound of the format against the fp32 reference math."""
import pytest
import torch

import oracle
from util import assert_bitexact, need_lib, rand_scales

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K", [(64, 512), (1000, 2048), (3, 32), (129, 384)])
def test_mx_activation_quantiser_bitexact(M, K):
    g = need_lib()
    gen = torch.Generator().manual_seed(M + K)
    x = (torch.randn(M, K, generator=gen) * torch.logspace(-3, 3, M)[:, None]).half()
    x[0, :32] = 0
    q_ref, s_ref = oracle.mx_block_quantize(x.float())
    q, s = g.mxfp8_quantize(x.cuda())
    assert_bitexact(s, s_ref, "E8M0 scale bytes")
    assert_bitexact(q, q_ref, "E4M3 elements")


@pytest.mark.parametrize("M,N,K", [(256, 2048, 512), (1000, 256, 512), (130, 160, 128)])
def test_dual_silu_mxfp8_output(M, N, K):
    g = need_lib()
    gen = torch.Generator().manual_seed(7 + M + N)
    A, sa = oracle.fp8_quantize_per_token(torch.randn(M, K, generator=gen))
    Wg = ((torch.rand(N, K, generator=gen) * 2 - 1) * 448).to(torch.float8_e4m3fn)
    Wu = ((torch.rand(N, K, generator=gen) * 2 - 1) * 448).to(torch.float8_e4m3fn)
    sbg, sbu = rand_scales(gen, N, 2e-4, 2e-3), rand_scales(gen, N, 2e-4, 2e-3)
    q, s = g.dual_gemm_fp8_silu_mxfp8(A.cuda(), Wg.cuda(), Wu.cuda(), sa.cuda(), sbg.cuda(), sbu.cuda())
    ref = oracle.fp8_dual_silu_ref(A, Wg, Wu, sa, sbg, sbu)
    got = oracle.mx_dequantize(q.cpu(), s.cpu())
    blk_amax = ref.reshape(M, N // 32, 32).abs().amax(-1, keepdim=True).expand(M, N // 32, 32).reshape(M, N)
    err = (got - ref).abs()
    # E4M3 carries 3 mantissa bits; a scaled block maximum in (448, 512) saturates: error <= 12.5 % of the block maximum
    assert bool((err <= 0.13 * blk_amax + 1e-6).all()), float((err / (blk_amax + 1e-12)).max())
    assert float((err / (blk_amax + 1e-12)).mean()) < 0.02
    # scale bytes follow the rule on the reference values except where the block maximum sits at a binade edge
    _, s_ref = oracle.mx_block_quantize(ref)
    assert float((s.cpu() != s_ref).float().mean()) < 0.01
    assert int((s.cpu().int() - s_ref.int()).abs().max()) <= 1
    # fused output == two-step path: the plain SwiGLU kernel's fp16 result dequantises to the same values within fp16 + e4m3 rounding
    h = g.dual_gemm_fp8_silu(A.cuda(), Wg.cuda(), Wu.cuda(), sa.cuda(), sbg.cuda(), sbu.cuda()).cpu().float()
    assert bool(((got - h).abs() <= 0.13 * blk_amax + 1e-3).all())


def tiled_ref(s, K):
    """CPU statement of the 128 x 4 scale tile order."""
    rows = s.shape[0]
    rb, kt = (rows + 127) // 128, K // 128
    out = torch.full((rb * kt * 512,), 127, dtype=torch.uint8)
    r = torch.arange(rows)[:, None]
    b = torch.arange(K // 32)[None, :]
    idx = ((r // 128) * kt + b // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + b % 4
    out[idx.reshape(-1)] = s.reshape(-1)
    return out


def test_scale_retiling():
    g = need_lib()
    gen = torch.Generator().manual_seed(4)
    for rows, K in [(128, 128), (300, 512), (5, 256)]:
        s = torch.randint(0, 255, (rows, K // 32), generator=gen, dtype=torch.uint8)
        got = g.mx_scales_to_tiled(s.cuda(), K)
        assert torch.equal(got.cpu(), tiled_ref(s, K))


def mx_operand(gen, rows, K, spread=True):
    v = torch.randn(rows, K, generator=gen)
    if spread:
        v = v * torch.logspace(-2, 2, K // 32).repeat_interleave(32)[None, :]     # different block magnitudes
    return oracle.mx_block_quantize(v)


# K <= 512 runs the weight-stationary kernel (256-column slices: N % 256 of 0, 128 and other remainders, 3 and 4
# K blocks, ragged M, more row blocks than one group walks), K = 2048 the streaming one
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (128, 128, 512), (300, 512, 512), (1000, 512, 2048), (64, 96, 256),
                                   (300, 384, 512), (257, 2048, 512), (200, 640, 384), (20000, 256, 512),
                                   (20000, 256, 640), (40000, 128, 1024)])   # streaming form, several tiles per CTA: both pipelines
def test_block_scaled_gemm(M, N, K):
    g = need_lib()
    gen = torch.Generator().manual_seed(M + N + K)
    Aq, As = mx_operand(gen, M, K)
    Wq, Ws = mx_operand(gen, N, K)
    c = g.gemm_mxfp8(Aq.cuda(), g.mx_scales_to_tiled(As.cuda(), K), Wq.cuda(), g.mx_scales_to_tiled(Ws.cuda(), K))
    ref = oracle.mx_gemm_ref(Aq, As, Wq, Ws)
    assert g.device_status()[0] == 0
    from util import assert_close
    assert_close(c, ref.half(), atol=float(ref.abs().max()) * 2 ** -9, rtol=2e-2, what="block-scaled GEMM")


@pytest.mark.parametrize("M,N,K", [(128, 64, 128), (256, 2048, 512), (1000, 192, 512), (300, 320, 512), (129, 2048, 256),
                                   (20000, 128, 384), (700, 256, 1024), (20000, 128, 640)])
def test_block_scaled_dual_silu(M, N, K):
    g = need_lib()
    gen = torch.Generator().manual_seed(3 * M + N + K)
    Aq, As = mx_operand(gen, M, K, spread=False)
    Wg = oracle.mx_block_quantize(torch.randn(N, K, generator=gen) * 0.05)
    Wu = oracle.mx_block_quantize(torch.randn(N, K, generator=gen) * 0.05)
    t = lambda s: g.mx_scales_to_tiled(s.cuda(), K)
    c = g.dual_gemm_mxfp8_silu(Aq.cuda(), t(As), Wg[0].cuda(), Wu[0].cuda(), t(Wg[1]), t(Wu[1]))
    ref = oracle.mx_dual_silu_ref(Aq, As, Wg[0], Wg[1], Wu[0], Wu[1])
    from util import assert_close
    assert_close(c, ref.half(), atol=float(ref.abs().max()) * 2 ** -9, rtol=2e-2, what="block-scaled SwiGLU")


def test_mx_ffn_chain():
    """fp8 SwiGLU emitting MXFP8 -> block-scaled down-projection consuming it (activation scales per 32 K)."""
    g = need_lib()
    gen = torch.Generator().manual_seed(77)
    M, D, F = 512, 512, 1024
    A, sa = oracle.fp8_quantize_per_token(torch.randn(M, D, generator=gen))
    Wg = ((torch.rand(F, D, generator=gen) * 2 - 1) * 448).to(torch.float8_e4m3fn)
    Wu = ((torch.rand(F, D, generator=gen) * 2 - 1) * 448).to(torch.float8_e4m3fn)
    sbg, sbu = rand_scales(gen, F, 2e-4, 2e-3), rand_scales(gen, F, 2e-4, 2e-3)
    Wd = oracle.mx_block_quantize(torch.randn(D, F, generator=gen) * 0.05)
    hq, hs = g.dual_gemm_fp8_silu_mxfp8(A.cuda(), Wg.cuda(), Wu.cuda(), sa.cuda(), sbg.cuda(), sbu.cuda())
    y = g.gemm_mxfp8(hq, g.mx_scales_to_tiled(hs, F), Wd[0].cuda(), g.mx_scales_to_tiled(Wd[1].cuda(), F))
    ref = oracle.mx_gemm_ref(hq.cpu(), hs.cpu(), Wd[0], Wd[1])         # oracle fed with the device's own MXFP8 activations
    from util import assert_close
    assert_close(y, ref.half(), atol=float(ref.abs().max()) * 2 ** -9, rtol=2e-2, what="MX down-projection")
