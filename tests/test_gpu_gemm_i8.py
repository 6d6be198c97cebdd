"""GPU parity: tcgen05 INT8 GEMMs through the C ABI vs the CPU oracle.

Integer accumulators and the dequant / rotary epilogues are compared bit for bit
against the arithmetic model; every fp16 result is also held to the reference's
own tolerance against the reference's fp32 host math."""
import pytest
import torch

import oracle
from conftest import load_golden
from util import T, assert_bitexact, assert_close, f16_equal_up_to_signed_zero, need_lib, rand_i8, rand_scales, rotary_rows

pytestmark = pytest.mark.gpu


def test_gemm_i32_golden():
    g = need_lib()
    gold = load_golden("gemm_i32")
    for tag in ("small", "full"):
        c = g.gemm_i8_i32(T(gold["a_" + tag]).cuda(), T(gold["b_" + tag]).cuda())
        assert_bitexact(c, T(gold["c_" + tag]), f"int32 accumulators ({tag}) vs reference golden")


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (128, 256, 512), (1, 8, 16), (127, 264, 144), (129, 512, 512),
                                   (300, 1536, 512), (1000, 512, 2048), (4096, 1536, 512), (256, 2048, 384)])
def test_gemm_i32_bitexact(M, N, K):
    g = need_lib()
    gen = torch.Generator().manual_seed(M * 131 + N * 17 + K)
    A, B = rand_i8(gen, M, K), rand_i8(gen, N, K)
    c = g.gemm_i8_i32(A.cuda(), B.cuda())
    assert_bitexact(c, oracle.gemm_i32(A, B), f"int32 accumulators {M}x{N}x{K}")


def test_gemm_i32_worst_case_magnitude():
    g = need_lib()
    A = torch.full((128, 2048), 127, dtype=torch.int8)
    B = torch.full((256, 2048), -127, dtype=torch.int8)
    B[::2] = 127
    c = g.gemm_i8_i32(A.cuda(), B.cuda())
    assert_bitexact(c, oracle.gemm_i32(A, B))


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (16384, 512, 512), (257, 520, 512), (64, 1536, 512), (2000, 512, 2048),
                                   (5000, 1536, 384), (3000, 4096, 512), (700, 1536, 640), (40000, 512, 1024)])
def test_gemm_dequant(M, N, K):
    """K <= 512 runs the weight-stationary schedule, larger K the streaming one."""
    g = need_lib()
    gen = torch.Generator().manual_seed(1000 + M + N + K)
    A, B = rand_i8(gen, M, K), rand_i8(gen, N, K)
    sa, sb = rand_scales(gen, M, 5e-3, 5e-2), rand_scales(gen, N)
    c = g.gemm_i8(A.cuda(), B.cuda(), sa.cuda(), sb.cuda())
    exact = oracle.gemm_dequant_exact(A, B, sa, sb)
    assert f16_equal_up_to_signed_zero(c, exact) == 0, "fp16 output differs from the exact-accumulator model"
    ref = oracle.gemm_dequant_ref(A, B, sa, sb)
    assert_close(c, ref.half(), atol=2 * float(ref.abs().max()) * 2 ** -11, rtol=1e-2, what="vs reference fp32 math")


def test_gemm_dequant_strided_views():
    g = need_lib()
    gen = torch.Generator().manual_seed(5)
    Abig, Bbig = rand_i8(gen, 200, 1024), rand_i8(gen, 264, 1024)
    A, B = Abig[:, 256:768], Bbig[:, :512]
    sa, sb = rand_scales(gen, 200), rand_scales(gen, 264)
    Cbig = torch.zeros(200, 512, dtype=torch.float16, device="cuda")
    out = Cbig[:, :264]
    g.gemm_i8(Abig.cuda()[:, 256:768], Bbig.cuda()[:, :512], sa.cuda(), sb.cuda(), out=out)
    exact = oracle.gemm_dequant_exact(A.contiguous(), B.contiguous(), sa, sb)
    assert f16_equal_up_to_signed_zero(out, exact) == 0
    assert float(Cbig[:, 264:].abs().max()) == 0.0, "wrote outside the N columns"


def test_rotary_reference_scenario():
    """The reference's own JIT parity case: M=64 (4x16), K=512, N=1536 (cute/test_gemm_i8_rotary_vs_openfish.py)."""
    g = need_lib()
    gold = load_golden("rotary")
    nhead, head_dim, rotary_dim, seqlen = (int(v) for v in gold["dims"])
    a, b, sa, sb, sn, cs = (T(gold[k]) for k in ("a", "b", "sa", "sb", "sin", "cos"))
    c = g.gemm_i8_rotary(a.cuda(), b.cuda(), sa.cuda(), sb.cuda(), sn.cuda(), cs.cuda(),
                         nhead, head_dim, rotary_dim, seqlen)
    ref16 = T(gold["c"]).half()
    err = (c.cpu().float() - ref16.float()).abs().max().item()
    assert err <= 0.05, f"max abs err {err} vs the reference's 0.05 gate"
    exact = oracle.rotary_exact(a, b, sa, sb, sn, cs, nhead, head_dim, rotary_dim, seqlen)
    assert f16_equal_up_to_signed_zero(c, exact) == 0


@pytest.mark.parametrize("M,seqlen,row_offset,K", [(256, 1024, 0, 512), (256, 333, 0, 512), (4096, 2048, 0, 512),
                                                   (1000, 2048, 1536, 512), (130, 16, 5, 512), (20000, 2048, 0, 512),
                                                   (4096, 2048, 0, 1024), (700, 77, 3, 640)])
def test_rotary_shapes(M, seqlen, row_offset, K):
    """K <= 512 runs the activation-stationary schedule, larger K the streaming one."""
    g = need_lib()
    nhead, head_dim, rotary_dim = 8, 64, 64
    N = 3 * nhead * head_dim
    gen = torch.Generator().manual_seed(2000 + M + seqlen)
    X = torch.randn(M, K, generator=gen)
    A, sa = oracle.quantize_tensor(X)
    B, sb = rand_i8(gen, N, K), rand_scales(gen, N)
    sn, cs = oracle.rope_tables(max(seqlen, 16), rotary_dim // 2, head_dim)
    c = g.gemm_i8_rotary(A.cuda(), B.cuda(), sa.cuda(), sb.cuda(), sn.cuda(), cs.cuda(),
                         nhead, head_dim, rotary_dim, seqlen, row_offset=row_offset)
    # the oracle indexes angle rows by m % seqlen: emulate the shard offset by prepending rows
    pad = row_offset
    Ap = torch.cat([torch.zeros(pad, K, dtype=torch.int8), A])
    sap = torch.cat([torch.ones(pad), sa])
    exact = oracle.rotary_exact(Ap, B, sap, sb, sn, cs, nhead, head_dim, rotary_dim, seqlen)[pad:]
    assert f16_equal_up_to_signed_zero(c, exact) == 0
    ref = oracle.rotary_ref(Ap, B, sap, sb, sn, cs, nhead, head_dim, rotary_dim, seqlen)[pad:]
    assert_close(c, ref.half(), atol=2 * float(ref.abs().max()) * 2 ** -11, rtol=1e-2, what="rotary vs reference math")


def test_rotary_identity_table_equals_plain_gemm():
    """sin=0, cos=1 must reproduce the plain dequant GEMM (the ROTARY_IDENTITY check of cute/main_rotary.cpp:99-103,
    gated there at 0.05 abs / 1 % rel).  The rotated columns apply the two scales in another order than the plain
    epilogue ((acc*sB)*(sA*1) against acc*(sA*sB)), so the two agree to one fp16 ulp, not bit for bit; the V
    columns are bit-identical, and the whole result equals the CPU model of the rotary epilogue bit for bit."""
    g = need_lib()
    gen = torch.Generator().manual_seed(9)
    A, B = rand_i8(gen, 256, 512), rand_i8(gen, 1536, 512)
    sa, sb = rand_scales(gen, 256), rand_scales(gen, 1536)
    sn, cs = torch.zeros(1024, 32), torch.ones(1024, 32)
    c = g.gemm_i8_rotary(A.cuda(), B.cuda(), sa.cuda(), sb.cuda(), sn.cuda(), cs.cuda(), 8, 64, 64, 1024)
    plain = g.gemm_i8(A.cuda(), B.cuda(), sa.cuda(), sb.cuda()).cpu()
    assert f16_equal_up_to_signed_zero(c[:, 1024:], plain[:, 1024:]) == 0
    assert_close(c, plain, atol=2e-7, rtol=2 ** -10, what="identity rotary vs plain GEMM (1 fp16 ulp)")
    exact = oracle.rotary_exact(A, B, sa, sb, sn, cs, 8, 64, 64, 1024)
    assert f16_equal_up_to_signed_zero(c, exact) == 0


def test_dual_silu_golden():
    g = need_lib()
    gold = load_golden("dual_silu")
    a, bg, bu, sa, sbg, sbu = (T(gold[k]) for k in ("a", "bg", "bu", "sa", "sbg", "sbu"))
    c = g.dual_gemm_i8_silu(a.cuda(), bg.cuda(), bu.cuda(), sa.cuda(), sbg.cuda(), sbu.cuda())
    ref = T(gold["c"])
    assert_close(c, ref.half(), atol=2 * float(ref.abs().max()) * 2 ** -11, rtol=1e-2, what="SwiGLU vs reference golden")


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 2048, 512), (4096, 2048, 512), (65, 136, 512), (9000, 2048, 512),
                                   (1000, 2048, 640), (4096, 1024, 768)])
def test_dual_silu_shapes(M, N, K):
    """K <= 512 runs the weight-stationary schedule, larger K the streaming one."""
    g = need_lib()
    gen = torch.Generator().manual_seed(3000 + M + N)
    X = torch.randn(M, K, generator=gen)
    A, sa = oracle.quantize_tensor(X)
    Bg, Bu = rand_i8(gen, N, K), rand_i8(gen, N, K)
    sbg, sbu = rand_scales(gen, N), rand_scales(gen, N)
    c = g.dual_gemm_i8_silu(A.cuda(), Bg.cuda(), Bu.cuda(), sa.cuda(), sbg.cuda(), sbu.cuda())
    model = oracle.dual_gemm_silu_model(A, Bg, Bu, sa, sbg, sbu)
    assert_close(c, model, atol=2 * float(model.float().abs().max()) * 2 ** -11, rtol=2e-3, what="vs kernel model")
    ref = oracle.dual_gemm_silu_ref(A, Bg, Bu, sa, sbg, sbu)
    assert_close(c, ref.half(), atol=2 * float(ref.abs().max()) * 2 ** -11, rtol=1e-2, what="vs reference math")


def test_ffn_chain_int8():
    """quantise -> dual GEMM SiLU -> re-quantise -> down-projection, each stage checked against the
    oracle fed with the device's own (bit-exact) intermediates so errors do not compound."""
    g = need_lib()
    gen = torch.Generator().manual_seed(4004)
    M, D, F = 1024, 512, 2048
    x = torch.randn(M, D, generator=gen).half()
    Wg, Wu, Wd = rand_i8(gen, F, D), rand_i8(gen, F, D), rand_i8(gen, D, F)
    sg, su, sd = rand_scales(gen, F), rand_scales(gen, F), rand_scales(gen, D)
    xq, xs = g.quantize_tensor(x.cuda())
    q_ref, s_ref = oracle.quantize_tensor(x.float())
    assert_bitexact(xq, q_ref); assert_bitexact(xs, s_ref)
    h = g.dual_gemm_i8_silu(xq, Wg.cuda(), Wu.cuda(), xs, sg.cuda(), su.cuda())
    ref_h = oracle.dual_gemm_silu_ref(q_ref, Wg, Wu, s_ref, sg, su)
    assert_close(h, ref_h.half(), atol=2 * float(ref_h.abs().max()) * 2 ** -11, rtol=1e-2, what="SwiGLU stage")
    hq, hs = g.quantize_tensor(h)
    hq_ref, hs_ref = oracle.quantize_tensor(h.cpu().float())
    assert_bitexact(hq, hq_ref); assert_bitexact(hs, hs_ref)
    y = g.gemm_i8(hq, Wd.cuda(), hs, sd.cuda())
    assert f16_equal_up_to_signed_zero(y, oracle.gemm_dequant_exact(hq_ref, Wd, hs_ref, sd)) == 0


def test_config2_full_size_sampled_rows():
    """BASELINE config 2 at full size (65536 tokens = 32 chunks x 2048 steps): rows are independent, so
    parity is checked on row blocks (first / middle / last tile, a ragged slice) against the oracle."""
    g = need_lib()
    nhead, head_dim, rotary_dim, seqlen, K = 8, 64, 64, 2048, 512
    M, N = 65536, 1536
    gen = torch.Generator().manual_seed(2001)
    x = torch.randn(M, K, generator=gen).half()
    B, sb = rand_i8(gen, N, K), rand_scales(gen, N)
    sn, cs = oracle.rope_tables(seqlen, 32, head_dim)
    xq, xs = g.quantize_tensor(x.cuda())
    c = g.gemm_i8_rotary(xq, B.cuda(), xs, sb.cuda(), sn.cuda(), cs.cuda(), nhead, head_dim, rotary_dim, seqlen)
    c = c.cpu()
    for lo, hi in [(0, 256), (32768 - 64, 32768 + 64), (65536 - 256, 65536), (12345, 12345 + 77)]:
        q_ref, s_ref = oracle.quantize_tensor(x[lo:hi].float())
        assert_bitexact(xq[lo:hi], q_ref)
        pad = lo % seqlen
        Ap = torch.cat([torch.zeros(pad, K, dtype=torch.int8), q_ref])
        sap = torch.cat([torch.ones(pad), s_ref])
        exact = oracle.rotary_exact(Ap, B, sap, sb, sn, cs, nhead, head_dim, rotary_dim, seqlen)[pad:]
        assert f16_equal_up_to_signed_zero(c[lo:hi], exact) == 0, f"rows {lo}:{hi}"


def test_bad_arguments_are_rejected_before_launch():
    g = need_lib()
    A = torch.zeros(128, 512, dtype=torch.int8, device="cuda")
    B = torch.zeros(256, 512, dtype=torch.int8, device="cuda")
    s = torch.ones(256, device="cuda")
    with pytest.raises(RuntimeError):
        g.gemm_i8(A[:, :500], B[:, :500], s, s)              # K % 16 != 0
    with pytest.raises(RuntimeError):
        g.gemm_i8(A[:, 8:264], B[:, 8:264], s, s)            # misaligned base
    sn = torch.zeros(16, 32, device="cuda")
    with pytest.raises(RuntimeError):
        g.gemm_i8_rotary(A, B, s, s, sn, sn, 8, 64, 64, 16)  # 2*nhead*head_dim > N
    sn48 = torch.zeros(16, 48, device="cuda")
    with pytest.raises(RuntimeError):
        g.gemm_i8_rotary(A, B, s, s, sn48, sn48, 1, 96, 96, 16)    # unsupported head_dim
    sn24 = torch.zeros(16, 24, device="cuda")
    with pytest.raises(RuntimeError):
        g.gemm_i8_rotary(A, B, s, s, sn24, sn24, 1, 64, 48, 16)    # unsupported rotary_dim
    with pytest.raises(RuntimeError):
        g.gemm_i8_rotary(A, B, s, s, sn48, sn48, 1, 64, 96, 16)    # rotary_dim > head_dim
    with pytest.raises(RuntimeError):
        g.gemm_i8(A.cpu(), B.cpu(), s.cpu(), s.cpu())        # no CPU path
    for bad_flags in (1, 2, 0x100, 0x200, 16):
        with pytest.raises(RuntimeError):
            g.gemm_i8(A, B, s, s, flags=bad_flags)           # diagnostic / unknown flag bits are not part of the ABI
    assert g.device_status()[0] == 0


def test_host_pipeline_equals_whole_batch_call():
    """Chunked upload / compute / download over three streams gives the bytes of one whole-batch call."""
    g = need_lib()
    from gigaslop_b200.hostpipe import QkvRotaryHostPipeline
    gen = torch.Generator().manual_seed(21)
    M, K, N, seqlen = 2500, 512, 1536, 333
    x = (torch.randn(M, K, generator=gen) * 3).half().pin_memory()
    W = rand_i8(gen, N, K).cuda()
    sw = rand_scales(gen, N).cuda()
    sn, cs = (t.cuda() for t in oracle.rope_tables(seqlen, 32, 64))
    q, s = g.quantize_tensor(x.cuda())
    whole = g.gemm_i8_rotary(q, W, s, sw, sn, cs, 8, 64, 64, seqlen, row_offset=7).cpu()
    out = torch.empty(M, N, dtype=torch.float16).pin_memory()
    pipe = QkvRotaryHostPipeline(M, K, N, "cuda", chunk_rows=1024, depth=2)
    for _ in range(2):                       # the second pass reuses every slot
        out.zero_()
        pipe.run(x, out, W, sw, sn, cs, 8, 64, 64, seqlen, row_offset=7)
        pipe.finish()
        assert_bitexact(out, whole, "host pipeline vs whole batch")
    # back-to-back passes without a join in between (the next pass starts under the download of this one), into two
    # result buffers; 2500 rows are three chunks, so the slots rotate across the passes
    out2 = torch.empty(M, N, dtype=torch.float16).pin_memory()
    out.zero_(); out2.zero_()
    for o in (out, out2, out):
        pipe.run(x, o, W, sw, sn, cs, 8, 64, 64, seqlen, row_offset=7, join=False)
    pipe.finish()
    assert_bitexact(out, whole, "pipelined passes, first buffer")
    assert_bitexact(out2, whole, "pipelined passes, second buffer")


@pytest.mark.parametrize("nhead,K,M,seqlen", [(6, 512, 700, 128), (1, 256, 300, 50), (3, 384, 1030, 2048), (12, 512, 260, 333)])
def test_rotary_other_head_counts(nhead, K, M, seqlen):
    """N = 3 * nhead * 64 that is not a multiple of the 256-column tile (tail tiles, rotated / V boundary inside a
    tile), K below four K blocks, sequence lengths that wrap inside a row block: bit for bit against the CPU model."""
    g = need_lib()
    head_dim = rotary_dim = 64
    N = 3 * nhead * head_dim
    gen = torch.Generator().manual_seed(nhead * 1000 + K + M)
    A, sa = oracle.quantize_tensor(torch.randn(M, K, generator=gen))
    B, sb = rand_i8(gen, N, K), rand_scales(gen, N)
    sn, cs = oracle.rope_tables(seqlen, rotary_dim // 2, head_dim)
    c = g.gemm_i8_rotary(A.cuda(), B.cuda(), sa.cuda(), sb.cuda(), sn.cuda(), cs.cuda(), nhead, head_dim, rotary_dim, seqlen)
    exact = oracle.rotary_exact(A, B, sa, sb, sn, cs, nhead, head_dim, rotary_dim, seqlen)
    assert f16_equal_up_to_signed_zero(c, exact) == 0
    assert g.device_status()[0] == 0


def test_stream_pipeline_equals_direct_calls():
    """Quantiser and GEMM of consecutive batches on two streams give the bytes of the two calls made one after the other."""
    g = need_lib()
    from gigaslop_b200.devpipe import QkvRotaryStreamPipeline
    gen = torch.Generator().manual_seed(33)
    M, K, N, seqlen = 3000, 512, 1536, 777
    W = rand_i8(gen, N, K).cuda()
    sw = rand_scales(gen, N).cuda()
    sn, cs = (t.cuda() for t in oracle.rope_tables(seqlen, 32, 64))
    xs = [(torch.randn(M, K, generator=gen) * (1 + i)).half().cuda() for i in range(7)]
    want = []
    for x in xs:
        q, s = g.quantize_tensor(x)
        want.append(g.gemm_i8_rotary(q, W, s, sw, sn, cs, 8, 64, 64, seqlen, row_offset=5).cpu())
    pipe = QkvRotaryStreamPipeline(M, K, N, "cuda")
    outs = [torch.empty(M, N, dtype=torch.float16, device="cuda") for _ in xs]
    for x, o in zip(xs, outs):                 # seven batches through three slots
        pipe.submit(x, o, W, sw, sn, cs, 8, 64, 64, seqlen, row_offset=5)
    pipe.finish()
    for i, (o, w_) in enumerate(zip(outs, want)):
        assert_bitexact(o.cpu(), w_, f"stream pipeline, batch {i}")
    assert g.device_status()[0] == 0


@pytest.mark.parametrize("steps,time_gemms", [(3, False), (5, 2), (7, True)])
def test_step_graph_equals_direct_calls(steps, time_gemms):
    """The step graph (quantiser + GEMM per batch, captured once, any number of steps, with or without event nodes
    around GEMMs) leaves the bytes of the direct calls in every output, and its events time real launches."""
    g = need_lib()
    from gigaslop_b200.devpipe import QkvRotaryGraph
    gen = torch.Generator().manual_seed(44)
    M, K, N, seqlen = 2000, 512, 1536, 333
    W = rand_i8(gen, N, K).cuda()
    sw = rand_scales(gen, N).cuda()
    sn, cs = (t.cuda() for t in oracle.rope_tables(seqlen, 32, 64))
    xs = [(torch.randn(M, K, generator=gen) * (1 + i)).half().cuda() for i in range(3)]
    want = []
    for x in xs:
        q, s = g.quantize_tensor(x)
        want.append(g.gemm_i8_rotary(q, W, s, sw, sn, cs, 8, 64, 64, seqlen, row_offset=9).cpu())
    outs = [torch.empty(M, N, dtype=torch.float16, device="cuda") for _ in xs]
    runner = QkvRotaryGraph(M, K, N, "cuda").capture(xs, outs, W, sw, sn, cs, 8, 64, 64, seqlen, row_offset=9,
                                                      steps=steps, time_gemms=time_gemms)
    assert runner.steps == steps
    for timed in ([False, True] if time_gemms else [False]):
        for o in outs:
            o.zero_()
        runner.replay(timed=timed)
        torch.cuda.synchronize()
        for i in range(min(steps, 3)):
            assert_bitexact(outs[i].cpu(), want[i], f"step graph, batch {i}, timed copy {timed}")
    if time_gemms:
        assert len(runner.gemm_events) == (steps if time_gemms is True else time_gemms)
        assert all(a_.elapsed_time(b_) > 0 for a_, b_ in runner.gemm_events)
    assert g.device_status()[0] == 0


@pytest.mark.parametrize("M,K,nhead,seqlen", [(300, 512, 8, 2048), (128, 128, 8, 64), (1000, 256, 3, 333), (2500, 384, 6, 100),
                                              (40000, 512, 8, 2048)])
def test_fused_quantise_rotary_equals_two_calls(M, K, nhead, seqlen):
    """fp16 activations quantised on chip inside the QKV + rotary GEMM: the bytes of quantize_tensor + gemm_i8_rotary
    (ragged M, 1 to 4 K pieces, several row blocks per CTA, N that is not a multiple of the tile) and the same scales."""
    g = need_lib()
    N = 3 * nhead * 64
    gen = torch.Generator().manual_seed(M + K + nhead)
    x = (torch.randn(M, K, generator=gen) * torch.logspace(-2, 2, M)[:, None]).half().cuda()
    x[M // 2] = 0                                            # an all-zero token: amax clamps to 1e-8
    W = rand_i8(gen, N, K).cuda()
    sw = rand_scales(gen, N).cuda()
    sn, cs = (t.cuda() for t in oracle.rope_tables(seqlen, 32, 64))
    q, s = g.quantize_tensor(x)
    want = g.gemm_i8_rotary(q, W, s, sw, sn, cs, nhead, 64, 64, seqlen, row_offset=3)
    s_out = torch.full((M,), -1.0, device="cuda")
    got = g.quantize_gemm_i8_rotary(x, W, sw, sn, cs, nhead, 64, 64, seqlen, row_offset=3, out_scale=s_out)
    assert g.device_status()[0] == 0
    assert_bitexact(s_out.cpu(), s.cpu(), "token scales of the fused kernel")
    assert_bitexact(got.cpu(), want.cpu(), "fused quantise + rotary GEMM vs two calls")
    # and against the CPU oracle (quantize_tensor, then the rotary epilogue on exact accumulators) on row slices
    xc, gc = x.cpu(), got.cpu()
    for lo, hi in [(0, min(M, 200)), (max(0, M // 2 - 70), min(M, M // 2 + 70)), (max(0, M - 130), M)]:
        q_ref, s_ref = oracle.quantize_tensor(xc[lo:hi].float())
        assert_bitexact(s_out[lo:hi].cpu(), s_ref, f"fused token scales vs oracle, rows {lo}:{hi}")
        exact = rotary_rows(oracle.rotary_exact, q_ref, s_ref, W.cpu(), sw.cpu(), sn.cpu(), cs.cpu(), nhead, 64, 64, seqlen, lo + 3)
        assert f16_equal_up_to_signed_zero(gc[lo:hi], exact) == 0, f"fused kernel vs oracle, rows {lo}:{hi}"


def test_sm_limit_changes_the_grid_not_the_result():
    """gsb200_set_sm_limit caps the persistent grids (here to 40 and 1 CTA): same bytes as with all SMs."""
    g = need_lib()
    from gigaslop_b200 import _lib
    L = _lib.lib()
    gen = torch.Generator().manual_seed(77)
    M, K, N, seqlen = 5000, 512, 1536, 300
    A, sa = oracle.quantize_tensor(torch.randn(M, K, generator=gen))
    W, sw = rand_i8(gen, N, K), rand_scales(gen, N)
    sn, cs = oracle.rope_tables(seqlen, 32, 64)
    args = (A.cuda(), W.cuda(), sa.cuda(), sw.cuda())
    want_r = g.gemm_i8_rotary(*args, sn.cuda(), cs.cuda(), 8, 64, 64, seqlen).cpu()
    want_d = g.gemm_i8(*args).cpu()
    try:
        for limit in (40, 1):
            assert L.gsb200_set_sm_limit(limit) == 0
            assert_bitexact(g.gemm_i8_rotary(*args, sn.cuda(), cs.cuda(), 8, 64, 64, seqlen).cpu(), want_r, f"rotary, {limit} SMs")
            assert_bitexact(g.gemm_i8(*args).cpu(), want_d, f"dequant, {limit} SMs")
        assert L.gsb200_set_sm_limit(-1) != 0
    finally:
        assert L.gsb200_set_sm_limit(0) == 0
    assert g.device_status()[0] == 0


@pytest.mark.parametrize("M", [19072, 20000, 25344])
def test_rotary_shared_leftover_row_blocks(M):
    """More row blocks than CTAs with an incomplete last round (1, 9 and 50 row blocks left over on 148 SMs): those
    row blocks are shared by 6, 6 and 2 CTAs.  Same bytes as the walk of a single CTA, which shares nothing (and which
    the small cases pin against the CPU model), and as 37 CTAs."""
    g = need_lib()
    from gigaslop_b200 import _lib
    L = _lib.lib()
    gen = torch.Generator().manual_seed(M)
    K, N, seqlen = 256, 1536, 1000
    A = torch.randint(-127, 128, (M, K), generator=gen, dtype=torch.int8).cuda()
    sa = (torch.rand(M, generator=gen) * 0.02).cuda()
    W, sw = rand_i8(gen, N, K).cuda(), rand_scales(gen, N).cuda()
    sn, cs = (t.cuda() for t in oracle.rope_tables(seqlen, 32, 64))
    got = g.gemm_i8_rotary(A, W, sa, sw, sn, cs, 8, 64, 64, seqlen, row_offset=11).cpu()
    # the shared row blocks are the last ones: they and the first block against the CPU model, bit for bit
    for lo, hi in [(0, 128), (M - 300, M)]:
        exact = rotary_rows(oracle.rotary_exact, A[lo:hi].cpu(), sa[lo:hi].cpu(), W.cpu(), sw.cpu(), sn.cpu(), cs.cpu(),
                            8, 64, 64, seqlen, lo + 11)
        assert f16_equal_up_to_signed_zero(got[lo:hi], exact) == 0, f"rows {lo}:{hi} vs oracle"
    try:
        for limit in (1, 37):
            assert L.gsb200_set_sm_limit(limit) == 0
            ref = g.gemm_i8_rotary(A, W, sa, sw, sn, cs, 8, 64, 64, seqlen, row_offset=11).cpu()
            assert_bitexact(got, ref, f"all SMs vs {limit}")
    finally:
        assert L.gsb200_set_sm_limit(0) == 0
    assert g.device_status()[0] == 0


def test_tensor_maps_are_cached_per_thread():
    """A launch on buffers this host thread has launched on before encodes no TMA tensor map (they are a pure function
    of pointer, shape and stride); a new output buffer costs exactly the one map that names it."""
    g = need_lib()
    L = g.lib()
    gen = torch.Generator().manual_seed(5)
    A, W = rand_i8(gen, 1000, 512).cuda(), rand_i8(gen, 1536, 512).cuda()
    sa, sw = rand_scales(gen, 1000).cuda(), rand_scales(gen, 1536).cuda()
    sn, cs = (t.cuda() for t in oracle.rope_tables(128, 32, 64))
    out = torch.empty(1000, 1536, dtype=torch.float16, device="cuda")
    first = g.gemm_i8_rotary(A, W, sa, sw, sn, cs, 8, 64, 64, 128, out=out).clone()
    n0 = int(L.gsb200_tensor_map_encodes())
    for _ in range(5):
        g.gemm_i8_rotary(A, W, sa, sw, sn, cs, 8, 64, 64, 128, out=out)
    assert int(L.gsb200_tensor_map_encodes()) == n0
    assert torch.equal(out, first)
    out2 = torch.empty_like(out)
    g.gemm_i8_rotary(A, W, sa, sw, sn, cs, 8, 64, 64, 128, out=out2)
    assert int(L.gsb200_tensor_map_encodes()) == n0 + 1
    assert torch.equal(out2, first)


@pytest.mark.parametrize("head_dim,rotary_dim,nhead,M,K,seqlen,row_offset",
                         [(128, 128, 4, 300, 512, 2048, 0), (128, 64, 2, 1000, 512, 333, 7), (64, 32, 8, 700, 256, 100, 0),
                          (128, 32, 1, 130, 384, 64, 0), (128, 96, 3, 2500, 512, 2048, 1536), (128, 128, 4, 700, 1024, 77, 0),
                          (64, 32, 5, 20000, 512, 2048, 0)])
def test_rotary_other_head_and_rotary_dims(head_dim, rotary_dim, nhead, M, K, seqlen, row_offset):
    """Heads of 128 columns and partially rotated heads (the columns of a head past rotary_dim pass through, as the V
    columns do): the general epilogue against the same exact-accumulator model, bit for bit."""
    g = need_lib()
    N = 3 * nhead * head_dim
    gen = torch.Generator().manual_seed(6000 + head_dim + rotary_dim + M)
    A, sa = oracle.quantize_tensor(torch.randn(M, K, generator=gen))
    B, sb = rand_i8(gen, N, K), rand_scales(gen, N)
    sn, cs = oracle.rope_tables(max(seqlen, 16), rotary_dim // 2, head_dim)
    c = g.gemm_i8_rotary(A.cuda(), B.cuda(), sa.cuda(), sb.cuda(), sn.cuda(), cs.cuda(), nhead, head_dim, rotary_dim, seqlen,
                         row_offset=row_offset)
    assert g.device_status()[0] == 0
    exact = rotary_rows(oracle.rotary_exact, A, sa, B, sb, sn, cs, nhead, head_dim, rotary_dim, seqlen, row_offset)
    assert f16_equal_up_to_signed_zero(c, exact) == 0
    ref = rotary_rows(oracle.rotary_ref, A, sa, B, sb, sn, cs, nhead, head_dim, rotary_dim, seqlen, row_offset)
    assert_close(c, ref.half(), atol=2 * float(ref.abs().max()) * 2 ** -11, rtol=1e-2, what="rotary vs reference math")
