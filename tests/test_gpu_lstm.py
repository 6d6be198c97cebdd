"""GPU checks of the persistent LSTM recurrence and the layer stack (full-rank sigmoid/tanh cell of the
benchmark stack: parity unpinned by the reference, the oracle is this repository's CPU statement with the
same rounding points).  Gate: the benchmark's rtol 2e-2, with an absolute floor because h and c live in [-1, 1] / O(1)
and cross zero (an element passes if abs err <= atol OR rel err <= 2e-2), plus a bound on the mean error."""
import pytest
import torch

import oracle
from util import assert_close, need_lib, rand_scales

pytestmark = pytest.mark.gpu


def make_layer(gen, H, C):
    W_ih = ((torch.rand(4 * H, C, generator=gen) * 2 - 1) * 0.1 * 448).to(torch.float8_e4m3fn)
    W_hh = ((torch.rand(4 * H, H, generator=gen) * 2 - 1) * 0.1 * 448).to(torch.float8_e4m3fn)
    s = torch.full((4 * H,), 1.0 / 448.0) * (0.9 + 0.2 * torch.rand(4 * H, generator=gen))
    s2 = torch.full((4 * H,), 1.0 / 448.0) * (0.9 + 0.2 * torch.rand(4 * H, generator=gen))
    b = 0.05 * torch.randn(4 * H, generator=gen)
    return dict(W_ih=W_ih, s_ih=s, b=b, W_hh=W_hh, s_hh=s2)


def cuda_layer(L):
    return {k: v.cuda() for k, v in L.items()}


def check_h(got, ref, what, tol=0.03, mean_tol=3e-3):
    assert_close(got, ref, atol=tol, rtol=2e-2, what=what)
    err = (got.float().cpu() - ref.float()).abs()
    assert float(err.mean()) <= mean_tol, f"{what}: mean abs err {float(err.mean())}"


@pytest.mark.parametrize("T,B,H,reverse,init", [(12, 130, 64, False, False), (40, 256, 384, True, True),
                                                (7, 128, 32, False, True), (25, 512, 384, False, False),
                                                # H > 384: the cooperative kernel (h through global scratch), four K blocks,
                                                # zero-padded K pieces of W and h when H % 128 != 0
                                                (10, 256, 512, False, True), (8, 130, 416, True, True),
                                                (20, 512, 512, True, False), (6, 300, 448, False, False)])
def test_recurrent_kernel_vs_oracle(T, B, H, reverse, init):
    g = need_lib()
    gen = torch.Generator().manual_seed(T * 7 + B + H)
    L = make_layer(gen, H, 64)
    ih = (torch.randn(T * B, 4 * H, generator=gen) * 0.5).half()
    h0 = ((torch.rand(B, H, generator=gen) * 2 - 1) * 448).to(torch.float8_e4m3fn) if init else None
    c0 = (torch.randn(B, H, generator=gen) * 0.3).half() if init else None
    r16, r8, rc = oracle.lstm_fullrank_recurrent_ref(ih, L["W_hh"], L["s_hh"], L["b"], T, B, reverse, h0, c0)
    h16, h8, c_last = g.lstm_layer(ih.cuda(), L["W_hh"].cuda(), L["s_hh"].cuda(), T, B, bias=L["b"].cuda(), reverse=reverse,
                                   h0=h0.cuda() if init else None, c0=c0.cuda() if init else None, want_c=True)
    torch.cuda.synchronize()
    assert g.device_status()[0] == 0
    check_h(h16, r16, "h fp16")
    check_h(h8.float() / 448.0, r8.float() / 448.0, "h e4m3", tol=0.05)
    check_h(c_last, rc, "final c", tol=0.05)


def test_two_layer_stack_vs_oracle():
    g = need_lib()
    gen = torch.Generator().manual_seed(55)
    T, B, C, H = 16, 128, 64, 128
    x = torch.randn(T * B, C, generator=gen)
    x8, sx = oracle.fp8_quantize_per_token(x)
    layers = [make_layer(gen, H, C), make_layer(gen, H, H)]
    ref = oracle.lstm_fullrank_stack_ref(x8, sx, layers, T, B, reverse_first=True)
    dl = [cuda_layer(L) for L in layers]
    out = g.lstm_stack(x8.cuda(), sx.cuda(), dl, T, B, reverse_first=True)
    check_h(out, ref, "stack output", tol=0.05, mean_tol=5e-3)
    # cut into time blocks, the next layer's projection on a second stream: the same bytes
    for nb in (3, 16):
        out2 = g.lstm_stack(x8.cuda(), sx.cuda(), dl, T, B, reverse_first=True, aux_stream=torch.cuda.Stream(), time_blocks=nb)
        torch.cuda.synchronize()
        assert torch.equal(out, out2), f"{nb} time blocks"
    assert g.device_status()[0] == 0


def test_three_layer_stack_h512_forward_first():
    """H = 512 (cooperative kernel), three layers, first layer forward, ragged batch."""
    g = need_lib()
    gen = torch.Generator().manual_seed(56)
    T, B, C, H = 9, 200, 128, 512
    x = torch.randn(T * B, C, generator=gen)
    x8, sx = oracle.fp8_quantize_per_token(x)
    layers = [make_layer(gen, H, C), make_layer(gen, H, H), make_layer(gen, H, H)]
    ref = oracle.lstm_fullrank_stack_ref(x8, sx, layers, T, B, reverse_first=False)
    dl = [cuda_layer(L) for L in layers]
    out = g.lstm_stack(x8.cuda(), sx.cuda(), dl, T, B, reverse_first=False)
    check_h(out, ref, "stack output", tol=0.05, mean_tol=5e-3)
    out2 = g.lstm_stack(x8.cuda(), sx.cuda(), dl, T, B, reverse_first=False, aux_stream=torch.cuda.Stream(), time_blocks=4)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
    assert g.device_status()[0] == 0


def test_long_sequence_drift():
    """2000 steps at H=384 (the benchmark's layer shape, one 128-row group): the error must stay bounded."""
    g = need_lib()
    gen = torch.Generator().manual_seed(2000)
    T, B, H = 2000, 128, 384
    L = make_layer(gen, H, 64)
    ih = (torch.randn(T * B, 4 * H, generator=gen) * 0.5).half()
    r16, _, rc = oracle.lstm_fullrank_recurrent_ref(ih, L["W_hh"], L["s_hh"], L["b"], T, B, False)
    h16, _, c_last = g.lstm_layer(ih.cuda(), L["W_hh"].cuda(), L["s_hh"].cuda(), T, B, bias=L["b"].cuda(), want_c=True)
    tail = slice((T - 50) * B, T * B)
    check_h(h16[tail], r16[tail], "h, last 50 steps", tol=0.06, mean_tol=5e-3)
    check_h(c_last, rc, "c after 2000 steps", tol=0.1, mean_tol=8e-3)


def test_lstm_rejects_unsupported_shapes():
    g = need_lib()
    ih = torch.zeros(4 * 8, 4 * 48, dtype=torch.float16, device="cuda")
    W = torch.zeros(4 * 48, 48, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    with pytest.raises(RuntimeError):
        g.lstm_layer(ih, W, torch.ones(4 * 48, device="cuda"), 4, 8)        # H % 32 != 0


@pytest.mark.parametrize("env_key", ["GSB200_LSTM_NO_CLUSTER", "GSB200_LSTM_ROWS128"])
def test_cluster_and_cooperative_kernels_agree(tmp_path, env_key):
    """The recurrence has three kernels: the cluster form on 64-row groups (the default while twice the CTAs fit the
    GPU), the cluster form on 128-row groups (h exchanged through distributed shared memory, H <= 384) and the
    cooperative form with global scratch (any H <= 512, and the fallback).  Same arithmetic per cell, so the same
    bytes: the other two forms are forced in a child process through the environment."""
    import os
    import subprocess
    import sys
    g = need_lib()
    T, B, H = 30, 300, 384
    gen = torch.Generator().manual_seed(77)
    L = make_layer(gen, H, 64)
    ih = (torch.randn(T * B, 4 * H, generator=gen) * 0.5).half()
    h0 = ((torch.rand(B, H, generator=gen) * 2 - 1) * 448).to(torch.float8_e4m3fn)
    inp = tmp_path / "in.pt"
    out = tmp_path / "out.pt"
    torch.save(dict(ih=ih, W=L["W_hh"], s=L["s_hh"], b=L["b"], h0=h0, T=T, B=B), inp)
    code = (
        "import sys, torch; sys.path.insert(0, %r); import gigaslop_b200 as g\n"
        "d = torch.load(%r)\n"
        "h16, h8, c = g.lstm_layer(d['ih'].cuda(), d['W'].cuda(), d['s'].cuda(), d['T'], d['B'], bias=d['b'].cuda(),\n"
        "                          h0=d['h0'].cuda(), want_c=True)\n"
        "torch.save(dict(h16=h16.cpu(), h8=h8.cpu().view(torch.uint8), c=c.cpu()), %r)\n"
    ) % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))), str(inp), str(out))
    env = dict(os.environ, **{env_key: "1"})
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    ref = torch.load(out)
    h16, h8, c = g.lstm_layer(ih.cuda(), L["W_hh"].cuda(), L["s_hh"].cuda(), T, B, bias=L["b"].cuda(), h0=h0.cuda(),
                              want_c=True)
    assert torch.equal(h16.cpu(), ref["h16"])
    assert torch.equal(h8.cpu().view(torch.uint8), ref["h8"])
    assert torch.equal(c.cpu(), ref["c"])
    assert g.device_status()[0] == 0


def test_gemm_sm_cap_does_not_reject_the_lstm():
    """gsb200_set_sm_limit caps the grids of the persistent GEMMs only: a layer whose 48 CTAs fit the GPU still runs
    (and gives the same bytes) while the cap is 40."""
    g = need_lib()
    L = g.lib()
    gen = torch.Generator().manual_seed(31)
    T, B, H = 5, 512, 384
    Lw = make_layer(gen, H, 64)
    ih = (torch.randn(T * B, 4 * H, generator=gen) * 0.5).half().cuda()
    args = (ih, Lw["W_hh"].cuda(), Lw["s_hh"].cuda(), T, B)
    want = g.lstm_layer(*args, bias=Lw["b"].cuda())[0]
    try:
        assert L.gsb200_set_sm_limit(40) == 0
        got = g.lstm_layer(*args, bias=Lw["b"].cuda())[0]
    finally:
        assert L.gsb200_set_sm_limit(0) == 0
    assert torch.equal(got, want)
    assert g.device_status()[0] == 0
