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
