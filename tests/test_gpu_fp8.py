"""GPU parity: FP8-E4M3 GEMM twins (kind::f8f6f4, fp32 accumulate) vs the CPU oracle.
Tolerance follows the reference: rtol 2e-2 with an absolute floor tied to the output range."""
import pytest
import torch

import oracle
from conftest import load_golden
from util import T, assert_close, need_lib, rand_scales

pytestmark = pytest.mark.gpu


def rand_e4m3(gen, *shape, amp=448.0):
    return ((torch.rand(shape, generator=gen) * 2 - 1) * amp).to(torch.float8_e4m3fn)


def test_fp8_all_ones_known_answer():
    """A = B = fp8(1.0), unit scales -> every C equals K (fly/main_rdna_fp8_gemm.cpp:136-205)."""
    g = need_lib()
    for M, N, K in [(128, 512, 512), (200, 264, 2048)]:
        A = torch.ones(M, K).to(torch.float8_e4m3fn).cuda()
        B = torch.ones(N, K).to(torch.float8_e4m3fn).cuda()
        c = g.gemm_fp8(A, B, torch.ones(M).cuda(), torch.ones(N).cuda())
        assert float((c.float() - K).abs().max()) <= 0.5


def test_fp8_gemm_golden():
    g = need_lib()
    gold = load_golden("fp8_gemm")
    aq = T(gold["aq"]).view(torch.float8_e4m3fn)
    w_nk = T(gold["wq_kn"]).view(torch.float8_e4m3fn).t().contiguous()
    c = g.gemm_fp8(aq.cuda(), w_nk.cuda(), T(gold["asc"]).cuda(), T(gold["ws"]).cuda())
    ref = T(gold["c_bf16_as_f32"])
    assert float((c.cpu().float() - ref).abs().max()) < 2.0          # fly/verify_fp8_gemm.py:85
    assert_close(c, ref, atol=float(ref.abs().max()) * 2 ** -7, rtol=2e-2, what="vs reference golden (bf16)")


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (1000, 512, 512), (333, 1536, 512), (256, 512, 2048), (64, 1536, 384)])
def test_fp8_gemm_random(M, N, K):
    g = need_lib()
    gen = torch.Generator().manual_seed(M + 3 * N + 7 * K)
    x = torch.randn(M, K, generator=gen)
    A, sa = oracle.fp8_quantize_per_token(x)
    W, sb = rand_e4m3(gen, N, K), rand_scales(gen, N)
    c = g.gemm_fp8(A.cuda(), W.cuda(), sa.cuda(), sb.cuda())
    ref = oracle.fp8_gemm_f16_ref(A, W, sa, sb)
    assert_close(c, ref.half(), atol=float(ref.abs().max()) * 2 ** -9, rtol=2e-2, what="fp8 GEMM vs fp32 reference")
    model = oracle.fp8_gemm_model(A, W, sa, sb)
    assert_close(c, model.half(), atol=float(ref.abs().max()) * 2 ** -10, rtol=4e-3, what="fp8 GEMM vs exact-sum model")


def test_fp8_rotary_reference_scenario():
    """M=64 (4x16), K=512, N=1536 as in fly/bench_fp8_gemm_rotary_vs_openfish.py, 0.05 abs gate (:148-151)."""
    g = need_lib()
    torch.manual_seed(0)
    nhead, head_dim, rotary_dim, seqlen, M, K = 8, 64, 64, 16, 64, 512
    N = 3 * nhead * head_dim
    A, sa = oracle.fp8_quantize_per_token(torch.randn(M, K) * 0.1)
    Wkn, sb = oracle.fp8_quantize_per_channel(torch.randn(K, N) * 0.1)
    W = Wkn.t().contiguous()
    sn, cs = oracle.rope_tables(seqlen, 32, head_dim)
    c = g.gemm_fp8_rotary(A.cuda(), W.cuda(), sa.cuda(), sb.cuda(), sn.cuda(), cs.cuda(), nhead, head_dim, rotary_dim, seqlen)
    ref = oracle.fp8_rotary_ref(A, W, sa, sb, sn, cs, nhead, head_dim, rotary_dim, seqlen)
    assert float((c.cpu().float() - ref.half().float()).abs().max()) <= 0.05


@pytest.mark.parametrize("M,seqlen", [(4096, 2048), (300, 333)])
def test_fp8_rotary_shapes(M, seqlen):
    g = need_lib()
    nhead, head_dim, rotary_dim, K = 8, 64, 64, 512
    N = 3 * nhead * head_dim
    gen = torch.Generator().manual_seed(77 + M)
    A, sa = oracle.fp8_quantize_per_token(torch.randn(M, K, generator=gen))
    W, sb = rand_e4m3(gen, N, K), rand_scales(gen, N)
    sn, cs = oracle.rope_tables(seqlen, 32, head_dim)
    c = g.gemm_fp8_rotary(A.cuda(), W.cuda(), sa.cuda(), sb.cuda(), sn.cuda(), cs.cuda(), nhead, head_dim, rotary_dim, seqlen)
    ref = oracle.fp8_rotary_ref(A, W, sa, sb, sn, cs, nhead, head_dim, rotary_dim, seqlen)
    assert_close(c, ref.half(), atol=float(ref.abs().max()) * 2 ** -9, rtol=2e-2, what="fp8 rotary")


@pytest.mark.parametrize("head_dim,rotary_dim,nhead,M,seqlen", [(128, 128, 4, 300, 2048), (128, 64, 2, 1000, 333), (64, 32, 8, 700, 100)])
def test_fp8_rotary_other_head_and_rotary_dims(head_dim, rotary_dim, nhead, M, seqlen):
    g = need_lib()
    K, N = 512, 3 * nhead * head_dim
    gen = torch.Generator().manual_seed(177 + M + head_dim)
    A, sa = oracle.fp8_quantize_per_token(torch.randn(M, K, generator=gen))
    W, sb = rand_e4m3(gen, N, K), rand_scales(gen, N)
    sn, cs = oracle.rope_tables(seqlen, rotary_dim // 2, head_dim)
    c = g.gemm_fp8_rotary(A.cuda(), W.cuda(), sa.cuda(), sb.cuda(), sn.cuda(), cs.cuda(), nhead, head_dim, rotary_dim, seqlen)
    ref = oracle.fp8_rotary_ref(A, W, sa, sb, sn, cs, nhead, head_dim, rotary_dim, seqlen)
    assert_close(c, ref.half(), atol=float(ref.abs().max()) * 2 ** -9, rtol=2e-2, what="fp8 rotary, general heads")


@pytest.mark.parametrize("M,N,K", [(256, 2048, 512), (1000, 256, 512), (64, 136, 128)])
def test_fp8_dual_silu(M, N, K):
    g = need_lib()
    gen = torch.Generator().manual_seed(99 + M + N)
    A, sa = oracle.fp8_quantize_per_token(torch.randn(M, K, generator=gen))
    Wg, Wu = rand_e4m3(gen, N, K), rand_e4m3(gen, N, K)
    sbg, sbu = rand_scales(gen, N, 2e-4, 2e-3), rand_scales(gen, N, 2e-4, 2e-3)
    c = g.dual_gemm_fp8_silu(A.cuda(), Wg.cuda(), Wu.cuda(), sa.cuda(), sbg.cuda(), sbu.cuda())
    ref = oracle.fp8_dual_silu_ref(A, Wg, Wu, sa, sbg, sbu)
    assert_close(c, ref.half(), atol=float(ref.abs().max()) * 2 ** -9, rtol=2e-2, what="fp8 SwiGLU")


def test_reference_style_python_interface():
    """Callers written against the reference's classes / compile_* factories."""
    g = need_lib()
    from gigaslop_b200 import compat
    gen = torch.Generator().manual_seed(12)
    M, N, K = 256, 512, 512
    A = torch.randint(-127, 128, (M, K), generator=gen, dtype=torch.int8)
    B = torch.randint(-127, 128, (N, K), generator=gen, dtype=torch.int8)
    sa, sb = rand_scales(gen, M), rand_scales(gen, N)
    C = torch.zeros(M, N, 1, dtype=torch.float16, device="cuda")
    compat.TensorOpGemmI8(None, None)(A.cuda()[:, :, None], B.cuda()[:, :, None], C, sa.cuda()[:, None], sb.cuda()[:, None])
    assert torch.equal(C[:, :, 0].cpu(), oracle.gemm_dequant_exact(A, B, sa, sb))
    launcher = compat.compile_fp8_gemm(M=M, N=N, K=K)
    A8, s8 = oracle.fp8_quantize_per_token(torch.randn(M, K, generator=gen))
    W8 = rand_e4m3(gen, N, K)
    C2 = torch.zeros(M, N, dtype=torch.float16, device="cuda")
    launcher(C2, A8.cuda(), W8.cuda(), s8.cuda(), sb.cuda(), torch.cuda.current_stream(), M)
    ref = oracle.fp8_gemm_f16_ref(A8, W8, s8, sb)
    assert_close(C2, ref.half(), atol=float(ref.abs().max()) * 2 ** -9, rtol=2e-2, what="compile_fp8_gemm launcher")
