"""The CPU oracle against the golden vectors produced by the reference's own
functions (tests/golden/make_golden.py).  Integer/byte results must be
bit-exact; fp32 results must be identical up to matmul summation order."""
import numpy as np
import torch

import oracle
from conftest import load_golden


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def test_quantize_tensor_bitexact():
    g = load_golden("quant_i8")
    q, s = oracle.quantize_tensor(T(g["x_f16"]).float())
    assert np.array_equal(q.numpy(), g["q"])
    assert np.array_equal(s.numpy().view(np.uint32), g["scale"].view(np.uint32))


def test_quantize_cpp_variant_differs_only_on_ties():
    g = load_golden("quant_i8")
    x = T(g["x_f16"]).float()
    q, s = oracle.quantize_tensor(x)
    qc, sc = oracle.quantize_per_row_cpp(x)
    diff = (q != qc)
    prod = x * (127.0 / x.abs().amax(-1).clamp_min(1e-8))[:, None]
    frac = (prod.abs() - prod.abs().floor())
    assert bool(((frac == 0.5) | ~diff).all())
    assert torch.equal(s, sc)


def test_gemm_i32_bitexact():
    g = load_golden("gemm_i32")
    for tag in ("small", "full"):
        c = oracle.gemm_i32(T(g["a_" + tag]), T(g["b_" + tag]))
        assert c.dtype == torch.int32
        assert np.array_equal(c.numpy(), g["c_" + tag])


def test_rotary_ref_matches_reference():
    g = load_golden("rotary")
    nhead, head_dim, rotary_dim, seqlen = (int(v) for v in g["dims"])
    c = oracle.rotary_ref(T(g["a"]), T(g["b"]), T(g["sa"]), T(g["sb"]), T(g["sin"]), T(g["cos"]),
                          nhead, head_dim, rotary_dim, seqlen)
    np.testing.assert_allclose(c.numpy(), g["c"], rtol=1e-5, atol=1e-6)
    s, co = oracle.rope_tables(seqlen, rotary_dim // 2, head_dim)
    assert np.array_equal(s.numpy(), g["sin"]) and np.array_equal(co.numpy(), g["cos"])
    # the exact-accumulator model agrees with the reference to fp16 resolution
    ce = oracle.rotary_exact(T(g["a"]), T(g["b"]), T(g["sa"]), T(g["sb"]), T(g["sin"]), T(g["cos"]),
                             nhead, head_dim, rotary_dim, seqlen)
    ref16 = T(g["c"]).to(torch.float16).float()
    assert (ce.float() - ref16).abs().max().item() <= 0.05          # cute/test_gemm_i8_rotary_vs_openfish.py:156


def test_dual_silu_ref_matches_reference():
    g = load_golden("dual_silu")
    args = [T(g[k]) for k in ("a", "bg", "bu", "sa", "sbg", "sbu")]
    c = oracle.dual_gemm_silu_ref(*args)
    np.testing.assert_allclose(c.numpy(), g["c"], rtol=1e-5, atol=1e-6)
    m = oracle.dual_gemm_silu_model(*args)
    ref = T(g["c"])
    err = (m.float() - ref).abs()
    assert bool(((err <= 2e-3) | (err <= 2e-3 * ref.abs())).all())


def test_fp8_quantisers_bitexact():
    g = load_golden("fp8_quant")
    q, s = oracle.fp8_quantize_per_token(T(g["x"]))
    assert np.array_equal(q.view(torch.uint8).numpy(), g["xq"])
    assert np.array_equal(s.numpy(), g["xs"])
    q, s = oracle.fp8_quantize_per_channel(T(g["w_kn"]))
    assert np.array_equal(q.view(torch.uint8).numpy(), g["wq"]) and np.array_equal(s.numpy(), g["ws"])
    q, s = oracle.fp8_quantize_scalar(T(g["w_kn"]))
    assert np.array_equal(q.view(torch.uint8).numpy(), g["sq"]) and np.array_equal(s.numpy(), g["ss"])


def test_software_e4m3_codec_matches_torch():
    b = np.arange(256, dtype=np.uint8)
    dec = oracle.e4m3_decode(b)
    tdec = torch.from_numpy(b).view(torch.float8_e4m3fn).float().numpy()
    ok = np.isnan(dec) == np.isnan(tdec)
    assert ok.all() and np.array_equal(dec[~np.isnan(dec)], tdec[~np.isnan(tdec)])
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.standard_normal(200000).astype(np.float32) * 100,
                        rng.standard_normal(50000).astype(np.float32) * 0.01,
                        np.linspace(-500, 500, 20001, dtype=np.float32),
                        dec[~np.isnan(dec)],
                        (dec[:-1] + dec[1:])[~np.isnan(dec[:-1] + dec[1:])] / 2])   # exact ties
    enc = oracle.e4m3_encode(x)
    tenc = torch.from_numpy(x).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    same = (enc == tenc) | ((enc & 0x7F) == 0) & ((tenc & 0x7F) == 0)    # +-0 both fine
    assert same.all(), np.flatnonzero(~same)[:10]


def test_fp8_gemm_ref_matches_reference():
    g = load_golden("fp8_gemm")
    aq = T(g["aq"]).view(torch.float8_e4m3fn)
    wkn = T(g["wq_kn"]).view(torch.float8_e4m3fn)
    c = oracle.naive_fp8_gemm_ref(aq, wkn, T(g["asc"]), T(g["ws"]))
    np.testing.assert_allclose(c.float().numpy(), g["c_bf16_as_f32"], rtol=1e-2, atol=1e-3)
    c2 = oracle.fp8_gemm_f16_ref(aq, wkn.t().contiguous(), T(g["asc"]), T(g["ws"]))
    np.testing.assert_allclose(c2.to(torch.bfloat16).float().numpy(), g["c_bf16_as_f32"], rtol=1e-2, atol=1e-3)
    c3 = oracle.fp8_gemm_model(aq, wkn.t().contiguous(), T(g["asc"]), T(g["ws"]))
    np.testing.assert_allclose(c3.numpy(), c2.numpy(), rtol=1e-4, atol=1e-5)


def test_factored_refs_match_reference():
    g = load_golden("factored_gemm")
    ih = oracle.factored_gemm_ref(T(g["x"]), T(g["dn"]), T(g["up"]), T(g["bias"]))
    np.testing.assert_allclose(ih.numpy(), g["ih"], rtol=1e-5, atol=1e-6)
    g = load_golden("factored_lstm")
    h, c = oracle.factored_lstm_step_ref(
        T(g["h_prev_q"]), T(g["dn_hh_fp8"]).view(torch.float8_e4m3fn), T(g["dn_hh_scale"]),
        T(g["up_hh"]), T(g["x_down"]), T(g["up_ih"]), T(g["bhh"]), T(g["bih"]), T(g["c"]))
    np.testing.assert_allclose(h.numpy(), g["h_ref"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(c.numpy(), g["c_ref"], rtol=1e-5, atol=1e-6)


def test_mx_roundtrip_properties():
    gen = torch.Generator().manual_seed(3)
    v = torch.randn(16, 256, generator=gen) * torch.logspace(-6, 6, 16)[:, None]
    v[0, :32] = 0
    q, s = oracle.mx_block_quantize(v)
    assert s.shape == (16, 8) and s.dtype == torch.uint8
    d = oracle.mx_dequantize(q, s)
    blk = v.reshape(16, 8, 32)
    amax = blk.abs().amax(-1, keepdim=True)
    err = (d.reshape(16, 8, 32) - blk).abs()
    assert bool((err <= amax * 2 ** -3 + 1e-30).all())       # e4m3: 3 mantissa bits, saturation <= 12.5 %
    assert s[0, 0].item() == 0
    # scaled block maximum lands in [256, 512)
    scaled = amax.squeeze(-1) / oracle.e8m0_decode(s)
    nz = amax.squeeze(-1) > 0
    assert bool(((scaled >= 256) & (scaled < 512))[nz].all())


def test_fp8_fused_refs_are_the_pinned_formulas():
    """``fp8_rotary_ref`` and ``fp8_dual_silu_ref`` restate inline script code of the reference
    (fly/bench_fp8_gemm_rotary_vs_openfish.py:91-122, fly/bench_fp8_dual_gemm_silu.py:62-68) for which no function
    could be executed to make a golden vector.  They are pinned through the pieces they are made of: the formula
    (dequantise, fp32 matmul, then rotate / silu * up) does not depend on the operand type, so fed with the INT8
    golden inputs they must reproduce the INT8 golden outputs made by the reference's own ``rotary_ref`` and
    ``dual_gemm_silu_ref``; and their matmul is ``fp8_gemm_f16_ref``, which the FP8 GEMM golden pins."""
    g = load_golden("rotary")
    nhead, head_dim, rotary_dim, seqlen = (int(v) for v in g["dims"])
    c = oracle.fp8_rotary_ref(T(g["a"]), T(g["b"]), T(g["sa"]), T(g["sb"]), T(g["sin"]), T(g["cos"]),
                              nhead, head_dim, rotary_dim, seqlen)
    np.testing.assert_allclose(c.numpy(), g["c"], rtol=1e-5, atol=1e-6)
    g = load_golden("dual_silu")
    c = oracle.fp8_dual_silu_ref(*[T(g[k]) for k in ("a", "bg", "bu", "sa", "sbg", "sbu")])
    np.testing.assert_allclose(c.numpy(), g["c"], rtol=1e-5, atol=1e-6)
    # on FP8 operands: the rotary reference is the pinned FP8 matmul followed by the pinned rotation, and with an
    # identity table it is that matmul
    g = load_golden("fp8_gemm")
    aq = T(g["aq"]).view(torch.float8_e4m3fn)
    w_nk = T(g["wq_kn"]).view(torch.float8_e4m3fn).t().contiguous()
    sa, sb = T(g["asc"]), T(g["ws"])
    w_nk, sb = torch.cat([w_nk.view(torch.uint8), w_nk.view(torch.uint8)[:64]]).view(torch.float8_e4m3fn), torch.cat([sb, sb[:64]])
    M, nh = aq.shape[0], 1                                # 192 weight rows = Q | K | V of one 64-wide head
    plain = oracle.fp8_gemm_f16_ref(aq, w_nk, sa, sb)
    ident = oracle.fp8_rotary_ref(aq, w_nk, sa, sb, torch.zeros(M, 32), torch.ones(M, 32), nh, 64, 64, M)
    assert torch.equal(ident, plain)
    sn, cs = oracle.rope_tables(M, 32, 64)
    rot = oracle.fp8_rotary_ref(aq, w_nk, sa, sb, sn, cs, nh, 64, 64, M)
    x0, x1 = plain[:, :32], plain[:, 32:64]
    assert torch.equal(rot[:, :32], x0 * cs - x1 * sn) and torch.equal(rot[:, 32:64], x0 * sn + x1 * cs)
    assert torch.equal(rot[:, 128:], plain[:, 128:])


def test_same_device_guard():
    """Host-side guard of the torch-facing layer: CPU tensors and tensors spread over several devices are refused
    before anything reaches the library (fake tensors: only ``.device`` is looked at)."""
    import types

    import pytest

    from gigaslop_b200.ops import same_device
    d0 = types.SimpleNamespace(device=torch.device("cuda", 0))
    d1 = types.SimpleNamespace(device=torch.device("cuda", 1))
    assert same_device(d0, None, d0) == torch.device("cuda", 0)
    assert same_device() is None
    with pytest.raises(ValueError):
        same_device(d0, d1)
    with pytest.raises(RuntimeError):
        same_device(d0, torch.zeros(1))
