"""GPU parity: per-token quantisers through the C ABI vs the CPU oracle (bit-exact)."""
import pytest
import torch

import oracle
from conftest import load_golden
from util import T, assert_bitexact, need_lib

pytestmark = pytest.mark.gpu


def test_int8_quantiser_golden():
    g = need_lib()
    gold = load_golden("quant_i8")
    x = T(gold["x_f16"]).cuda()
    q, s = g.quantize_tensor(x)
    assert_bitexact(q, T(gold["q"]), "int8 values vs reference golden")
    assert_bitexact(s, T(gold["scale"]), "scales vs reference golden")
    q32, s32 = g.quantize_tensor(x.float())
    assert_bitexact(q32, T(gold["q"]), "fp32-input path")
    assert_bitexact(s32, T(gold["scale"]), "fp32-input path scales")


@pytest.mark.parametrize("M,K", [(16384, 512), (1, 512), (129, 2048), (777, 384), (33, 1024), (5, 8), (64, 4096 + 64)])
def test_int8_quantiser_bitexact(M, K):
    g = need_lib()
    gen = torch.Generator().manual_seed(1001)
    x = torch.randn(M, K, generator=gen).half()
    q_ref, s_ref = oracle.quantize_tensor(x.float())
    q, s = g.quantize_tensor(x.cuda())
    assert_bitexact(q, q_ref, f"int8 [{M},{K}]")
    assert_bitexact(s, s_ref, f"scale [{M},{K}]")


def test_int8_quantiser_strided_and_empty():
    g = need_lib()
    gen = torch.Generator().manual_seed(7)
    big = torch.randn(100, 1024, generator=gen).half().cuda()
    view = big[:, :512]                       # row stride 1024
    q, s = g.quantize_tensor(view)
    q_ref, s_ref = oracle.quantize_tensor(view.cpu().float())
    assert_bitexact(q, q_ref)
    assert_bitexact(s, s_ref)
    q0, s0 = g.quantize_tensor(torch.empty(0, 512, dtype=torch.float16, device="cuda"))
    assert q0.shape == (0, 512) and s0.shape == (0,)


def test_int8_requant_of_swiglu_shaped_activations():
    g = need_lib()
    gen = torch.Generator().manual_seed(3003)
    x = (torch.randn(4096, 2048, generator=gen) * 3).half()
    q_ref, s_ref = oracle.quantize_tensor(x.float())
    q, s = g.quantize_tensor(x.cuda())
    assert_bitexact(q, q_ref)
    assert_bitexact(s, s_ref)


@pytest.mark.parametrize("torch_form", [True, False])
@pytest.mark.parametrize("M,K", [(48, 256), (1000, 512), (130, 2048), (9, 384)])
def test_fp8_quantiser_bitexact(M, K, torch_form):
    g = need_lib()
    gen = torch.Generator().manual_seed(1005)
    x = torch.randn(M, K, generator=gen).half()
    x[0] = 0
    if M > 4:
        x[4] *= 300
    fn = oracle.fp8_quantize_per_token if torch_form else oracle.fp8_quantize_per_token_kernel
    q_ref, s_ref = fn(x.float())
    q, s = g.fp8_quantize_per_token(x.cuda(), torch_formulation=torch_form)
    assert_bitexact(s, s_ref, "fp8 scale")
    assert_bitexact(q, q_ref, "fp8 bytes")


def test_fp8_quantiser_golden():
    g = need_lib()
    gold = load_golden("fp8_quant")
    q, s = g.fp8_quantize_per_token(T(gold["x"]).cuda(), torch_formulation=True)
    assert_bitexact(q.view(torch.uint8), T(gold["xq"]), "fp8 bytes vs reference golden")
    assert_bitexact(s, T(gold["xs"]), "fp8 scales vs reference golden")


def test_bounded_wait_gives_up_and_reports():
    """A wait nothing satisfies must end by itself and leave a code in the status word."""
    g = need_lib()
    L = g.lib()
    assert g.device_status()[0] == 0
    assert L.gsb200_set_spin_budget(200000) == 0          # ~0.1 ms of SM clocks
    try:
        assert L.gsb200_selftest_wait_timeout(None) == 0
        torch.cuda.synchronize()
        st = g.device_status()
        assert st[0] & 4 and st[1] == 0xdead
        assert g.device_status()[0] == 0                    # read clears
    finally:
        assert L.gsb200_set_spin_budget(0) == 0
    x = torch.randn(64, 512).half().cuda()                  # context still healthy
    q, s = g.quantize_tensor(x)
    q_ref, _ = oracle.quantize_tensor(x.cpu().float())
    assert torch.equal(q.cpu(), q_ref)
