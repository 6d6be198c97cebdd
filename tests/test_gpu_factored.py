"""GPU parity of the low-rank ("factored") LSTM pieces against the reference's own host references
(golden vectors from fly/bench_factored_lstm.py make_inputs()/reference(), tolerance 0.08 abs as at :100)."""
import pytest
import torch

import oracle
from conftest import load_golden
from util import T, assert_close, need_lib

pytestmark = pytest.mark.gpu


def test_factored_lstm_step_golden():
    g = need_lib()
    gd = load_golden("factored_lstm")
    h_prev8 = T(gd["h_prev_fp8"]).view(torch.float8_e4m3fn)
    dn8 = T(gd["dn_hh_fp8"]).view(torch.float8_e4m3fn)              # [K_hh, H]
    B, H = h_prev8.shape
    sx = torch.full((B,), 1.0 / 448.0)
    # recurrent down-projection exactly as the pipeline runs it (fp8 h_prev, scalar-scaled fp8 weights)
    hh_down = g.fp8_down_proj(h_prev8.cuda(), sx.cuda(), dn8.cuda(), T(gd["dn_hh_scale"]).cuda())
    ref_down = oracle.down_proj_ref(h_prev8, sx, dn8, T(gd["dn_hh_scale"]))
    assert_close(hh_down, ref_down.half(), atol=2e-3, rtol=2e-2, what="fp8 down-projection")
    c = T(gd["c"]).clone().cuda()
    h8 = torch.zeros(B, H, dtype=torch.uint8, device="cuda")
    g.factored_lstm_step(h8, c, hh_down, T(gd["up_hh"]).half().cuda(), T(gd["bhh"]).cuda(),
                         T(gd["x_down"]).cuda(), T(gd["up_ih"]).half().cuda(), T(gd["bih"]).cuda())
    h = h8.view(torch.float8_e4m3fn).float().cpu() / 448.0
    assert float((h - T(gd["h_ref"])).abs().max()) < 0.08
    assert float((c.cpu() - T(gd["c_ref"])).abs().max()) < 0.08
    assert float((c.cpu() - T(gd["c_ref"])).abs().mean()) < 2e-3


@pytest.mark.parametrize("B", [64, 512, 200])
def test_factored_lstm_step_reference_shape(B):
    """H=1024, K_hh=R=128 as deployed (fly/export_configs/rdna_fp8_factored_lstm.toml)."""
    g = need_lib()
    H, K, R = 1024, 128, 128
    gen = torch.Generator().manual_seed(42 + B)
    h_prev = (torch.rand(B, H, generator=gen) * 2 - 1) * 0.5
    h8 = (h_prev * 448).clamp(-448, 448).to(torch.float8_e4m3fn)
    dn_hh = torch.randn(K, H, generator=gen) * 0.1
    dn8, dn_s = oracle.fp8_quantize_scalar(dn_hh)
    up_hh = torch.randn(4 * H, K, generator=gen) * 0.1
    up_ih = torch.randn(4 * H, R, generator=gen) * 0.1
    bhh, bih = torch.randn(4 * H, generator=gen) * 0.05, torch.randn(4 * H, generator=gen) * 0.05
    x_down = (torch.randn(B, R, generator=gen) * 0.3).half()
    c0 = torch.randn(B, H, generator=gen) * 0.1
    h_ref, c_ref = oracle.factored_lstm_step_ref(h8.float() / 448.0, dn8, dn_s, up_hh, x_down, up_ih, bhh, bih, c0)
    sx = torch.full((B,), 1.0 / 448.0).cuda()
    hh_down = g.fp8_down_proj(h8.cuda(), sx, dn8.cuda(), dn_s.cuda())
    c = c0.clone().cuda()
    out = torch.zeros(B, H, dtype=torch.uint8, device="cuda")
    g.factored_lstm_step(out, c, hh_down, up_hh.half().cuda(), bhh.cuda(), x_down.cuda(), up_ih.half().cuda(), bih.cuda())
    h = out.view(torch.float8_e4m3fn).float().cpu() / 448.0
    assert float((h - h_ref).abs().max()) < 0.08 and float((c.cpu() - c_ref).abs().max()) < 0.08
    assert g.device_status()[0] == 0


@pytest.mark.parametrize("M", [64, 8200, 1])
def test_f16_down_proj(M):
    g = need_lib()
    gen = torch.Generator().manual_seed(M)
    x = (torch.randn(M, 1024, generator=gen) * 0.1).half()
    dn = (torch.randn(128, 1024, generator=gen) * 0.1).half()
    out = g.gemm_f16(x.cuda(), dn.cuda())
    ref = x.float() @ dn.float().t()
    assert_close(out, ref.half(), atol=float(ref.abs().max()) * 2 ** -9, rtol=1e-2, what="f16 down-projection")


def test_factored_gemm_chain_matches_reference_golden():
    """ih = (x . dn^T) . up^T + bias (fly/bench_factored_gemm.py:54-55) built from the two device GEMMs;
    rel < 0.08 as the reference gates small M (:60-66)."""
    g = need_lib()
    gd = load_golden("factored_gemm")
    x, dn, up, bias = (T(gd[k]) for k in ("x", "dn", "up", "bias"))
    x8, sx = oracle.fp8_quantize_per_token(x)
    dn8, sdn = oracle.fp8_quantize_scalar(dn)
    x_down = g.fp8_down_proj(x8.cuda(), sx.cuda(), dn8.cuda(), sdn.cuda())
    ih = g.gemm_f16(x_down, up.half().cuda()).float().cpu() + bias
    ref = T(gd["ih"])
    assert float((ih - ref).abs().max() / ref.abs().max()) < 0.08


@pytest.mark.parametrize("M", [256, 1000, 1])
def test_fused_factored_gemm_entry_point(M):
    """gsb200_fac_gemm_fp8_f16 (one call, no scratch: the fp16 intermediate lives inside the output) against the
    reference's fp32 chain (fly/bench_factored_gemm.py:54-55, rel < 0.08) and, tightly, against the same two
    rounding points done on the CPU."""
    g = need_lib()
    gen = torch.Generator().manual_seed(100 + M)
    C, R, N = 1024, 128, 4096
    x = torch.randn(M, C, generator=gen) * 0.1
    dn = torch.randn(R, C, generator=gen) * 0.1
    up = (torch.randn(N, R, generator=gen) * 0.1).half()
    bias = torch.randn(N, generator=gen) * 0.05
    x8, sx = oracle.fp8_quantize_per_token(x)
    dn8, sdn = oracle.fp8_quantize_scalar(dn)
    ih = g.fp8_factored_gemm(x8.cuda(), sx.cuda(), dn8.cuda(), sdn.cuda(), up.cuda(), bias.cuda()).float().cpu()
    ref = oracle.factored_gemm_ref(x, dn, up.float(), bias)
    assert float((ih - ref).abs().max() / ref.abs().max()) < 0.08
    x_down = oracle.down_proj_ref(x8, sx, dn8, sdn).half()
    model = (x_down.double() @ up.double().t()).float() + bias
    assert_close(ih, model.half().float(), atol=float(model.abs().max()) * 2 ** -9, rtol=1e-2, what="fused factored GEMM")
    # the two-call form gives the same bytes
    two = g.gemm_f16(g.fp8_down_proj(x8.cuda(), sx.cuda(), dn8.cuda(), sdn.cuda()), up.cuda()).float().cpu()
    assert float(((two + bias).half().float() - ih).abs().max()) <= float(model.abs().max()) * 2 ** -9


@pytest.mark.parametrize("M,C,R,N", [(500, 512, 64, 1000), (130, 256, 256, 264), (3000, 1024, 128, 1536)])
def test_fused_factored_gemm_other_shapes(M, C, R, N):
    """Other ranks and widths (N not a multiple of the tile, R = 256 = the largest resident x_down, R = 64)."""
    g = need_lib()
    gen = torch.Generator().manual_seed(M + C + R + N)
    x = torch.randn(M, C, generator=gen) * 0.1
    dn = torch.randn(R, C, generator=gen) * 0.1
    up = (torch.randn(N, R, generator=gen) * 0.1).half()
    bias = torch.randn(N, generator=gen) * 0.05
    x8, sx = oracle.fp8_quantize_per_token(x)
    dn8, sdn = oracle.fp8_quantize_scalar(dn)
    ih = g.fp8_factored_gemm(x8.cuda(), sx.cuda(), dn8.cuda(), sdn.cuda(), up.cuda(), bias.cuda()).float().cpu()
    x_down = oracle.down_proj_ref(x8, sx, dn8, sdn).half()
    model = (x_down.double() @ up.double().t()).float() + bias
    assert_close(ih, model.half().float(), atol=float(model.abs().max()) * 2 ** -9, rtol=1e-2, what="fused factored GEMM")
    assert g.device_status()[0] == 0
