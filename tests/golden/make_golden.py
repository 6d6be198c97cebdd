"""Generate the golden vectors under tests/golden/ by running the reference's OWN
host-side functions on small seeded inputs.

The reference's scripts cannot be imported as modules (they build CUDA tensors
or import an AMD-only DSL at import time), so each needed function definition
is located in the reference file by name with ``ast`` and executed in a scratch
namespace -- the code that runs is the reference's, unmodified, read from the
reference checkout at generation time.  Nothing of it is stored in the
fixtures except inputs and outputs.

Usage (only where the reference checkout exists):
    python tests/golden/make_golden.py /path/to/reference
"""
import ast
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_functions(path, names, extra_globals=None):
    """Exec only the named top-level function defs of ``path``; return namespace."""
    src = open(path).read()
    tree = ast.parse(src)
    ns = {"torch": torch, "__name__": "golden_extract"}
    ns.update(extra_globals or {})
    wanted = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    missing = set(names) - {n.name for n in wanted}
    if missing:
        raise RuntimeError(f"{path}: functions not found: {sorted(missing)}")
    mod = ast.Module(body=wanted, type_ignores=[])
    exec(compile(mod, path, "exec"), ns)
    return ns


def u8(t):
    return t.view(torch.uint8).numpy()


def main(ref):
    torch.set_num_threads(1)
    cute = os.path.join(ref, "cute")
    fly = os.path.join(ref, "fly")
    out = {}

    # ---- 1. INT8 per-token quantiser -------------------------------------
    q_ns = load_functions(os.path.join(cute, "bench_quant_i8.py"), ["quantize_tensor"])
    g = torch.Generator().manual_seed(1001)
    X = torch.randn(96, 512, generator=g).half()
    X[3] = 0                                   # all-zero row -> eps clamp
    X[5, :] = torch.linspace(-3, 3, 512).half()
    X[7, :8] = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 127.0, -127.0]).half()  # ties at qs==1
    X[9] *= 1000.0
    X[11] *= 1e-4
    qi, qs = q_ns["quantize_tensor"](X.float(), dim=-1)
    out["quant_i8"] = dict(x_f16=X.numpy(), q=qi.numpy(), scale=qs.numpy())

    # ---- 2. int32 GEMM ----------------------------------------------------
    g_ns = load_functions(os.path.join(cute, "ampere_gemm_i8.py"), ["gemm_ref"])
    g = torch.Generator().manual_seed(1002)
    A2 = torch.randint(-2, 3, (40, 128), generator=g, dtype=torch.int8)
    B2 = torch.randint(-2, 3, (48, 128), generator=g, dtype=torch.int8)
    A3 = torch.randint(-127, 128, (40, 128), generator=g, dtype=torch.int8)
    B3 = torch.randint(-127, 128, (48, 128), generator=g, dtype=torch.int8)

    def run_gemm_ref(A, B):
        # called the way the reference's run() does: (L,M,K) x (L,K,N) int32 on CPU
        # (cute/ampere_gemm_i8.py:838-840)
        r = g_ns["gemm_ref"](A.to(torch.int32)[None], B.to(torch.int32).t()[None])
        return r[0].to(torch.int32)
    out["gemm_i32"] = dict(a_small=A2.numpy(), b_small=B2.numpy(), c_small=run_gemm_ref(A2, B2).numpy(),
                           a_full=A3.numpy(), b_full=B3.numpy(), c_full=run_gemm_ref(A3, B3).numpy())

    # ---- 3. QKV + rotary (the reference's M=64 / seq=16 scenario) ---------
    r_ns = load_functions(os.path.join(cute, "ampere_gemm_i8_rotary.py"), ["rotary_ref"])
    torch.manual_seed(0)
    nhead, head_dim, rotary_dim, seqlen = 8, 64, 64, 16
    M, K, N = 64, 512, 3 * nhead * head_dim
    A_f = torch.randn(M, K) * 0.1
    B_f = torch.randn(N, K) * 0.1
    A8, sa = q_ns["quantize_tensor"](A_f, dim=-1)
    B8, sb = q_ns["quantize_tensor"](B_f, dim=-1)
    rh = rotary_dim // 2
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, rh).float() / head_dim * 2))
    freqs = torch.outer(torch.arange(seqlen).float(), inv_freq)
    sin_b, cos_b = freqs.sin().contiguous(), freqs.cos().contiguous()
    C = r_ns["rotary_ref"](A8, B8, sa, sb, sin_b, cos_b, nhead, head_dim, rotary_dim, seqlen)
    out["rotary"] = dict(a=A8.numpy(), b=B8.numpy(), sa=sa.numpy(), sb=sb.numpy(),
                         sin=sin_b.numpy(), cos=cos_b.numpy(), c=C.numpy(),
                         dims=np.array([nhead, head_dim, rotary_dim, seqlen]))

    # ---- 4. dual GEMM + SiLU ----------------------------------------------
    d_ns = load_functions(os.path.join(cute, "ampere_dual_gemm_i8_silu.py"), ["dual_gemm_silu_ref"])
    torch.manual_seed(42)
    A_f = torch.randn(64, 512)
    Bg_f = torch.randn(256, 512) * 0.05
    Bu_f = torch.randn(256, 512) * 0.05
    A8, sa = q_ns["quantize_tensor"](A_f)
    Bg8, sbg = q_ns["quantize_tensor"](Bg_f)
    Bu8, sbu = q_ns["quantize_tensor"](Bu_f)
    C = d_ns["dual_gemm_silu_ref"](A8, Bg8, Bu8, sa, sbg, sbu)
    out["dual_silu"] = dict(a=A8.numpy(), bg=Bg8.numpy(), bu=Bu8.numpy(), sa=sa.numpy(),
                            sbg=sbg.numpy(), sbu=sbu.numpy(), c=C.numpy())

    # ---- 5. FP8 quantisers + pre-shuffle ----------------------------------
    f_ns = load_functions(os.path.join(fly, "rdna_fp8_preshuffle_gemm.py"),
                          ["fp8_quantize_per_token", "fp8_quantize_per_channel", "preshuffle_b_fp8"])
    s_ns = load_functions(os.path.join(fly, "rdna_fp8_factored_gemm.py"),
                          ["fp8_quantize_scalar", "preshuffle_b_f16"], {"FP8_MAX": 448.0})
    g = torch.Generator().manual_seed(1005)
    Xf = torch.randn(48, 256, generator=g).half().float()
    Xf[2] = 0
    Xf[4] *= 300.0
    xq, xs = f_ns["fp8_quantize_per_token"](Xf)
    Wkn = torch.randn(256, 128, generator=g) * 0.1
    wq, ws = f_ns["fp8_quantize_per_channel"](Wkn)
    sq, ss = s_ns["fp8_quantize_scalar"](Wkn)
    out["fp8_quant"] = dict(x=Xf.numpy(), xq=u8(xq), xs=xs.numpy(), w_kn=Wkn.numpy(), wq=u8(wq),
                            ws=ws.numpy(), sq=u8(sq), ss=ss.numpy(),
                            w_shuf=f_ns["preshuffle_b_fp8"](wq).numpy(),
                            w_shuf_f16=s_ns["preshuffle_b_f16"](Wkn.half()).numpy())

    # ---- 6. FP8 GEMM ------------------------------------------------------
    v_ns = load_functions(os.path.join(fly, "verify_fp8_gemm.py"), ["naive_fp8_gemm_ref"])
    A_f = torch.randn(32, 256, generator=g) * 0.1
    aq, asc = f_ns["fp8_quantize_per_token"](A_f)
    Cb = v_ns["naive_fp8_gemm_ref"](aq, wq, asc, ws)
    out["fp8_gemm"] = dict(aq=u8(aq), asc=asc.numpy(), wq_kn=u8(wq), ws=ws.numpy(), c_bf16_as_f32=Cb.float().numpy())

    # ---- 7. factored GEMM reference ---------------------------------------
    fg_ns = load_functions(os.path.join(fly, "bench_factored_gemm.py"), ["ref_rows"])
    Cc, Rr, Nn = 128, 32, 256
    dn = torch.randn(Rr, Cc, generator=g) * 0.1
    up = torch.randn(Nn, Rr, generator=g) * 0.1
    bias = torch.randn(Nn, generator=g) * 0.05
    xr = torch.randn(40, Cc, generator=g) * 0.1
    out["factored_gemm"] = dict(x=xr.numpy(), dn=dn.numpy(), up=up.numpy(), bias=bias.numpy(),
                                ih=fg_ns["ref_rows"](xr, dict(dn=dn, up=up, bias=bias)).numpy())

    # ---- 8. factored LSTM step (reference make_inputs + reference, shrunk) -
    Hh, Kh, Rr = 128, 64, 64
    l_glob = dict(H=Hh, K_HH=Kh, R=Rr, FH=4 * Hh, OUT_SCALE=1.0 / 448.0,
                  fp8_quantize_scalar=s_ns["fp8_quantize_scalar"],
                  preshuffle_b_fp8=f_ns["preshuffle_b_fp8"],
                  preshuffle_b_f16=s_ns["preshuffle_b_f16"])
    l_ns = load_functions(os.path.join(fly, "bench_factored_lstm.py"), ["make_inputs", "reference"], l_glob)
    inp = l_ns["make_inputs"](32, "cpu")
    h_ref, c_ref = l_ns["reference"](inp)
    out["factored_lstm"] = dict(
        h_prev_q=inp["h_prev_q"].numpy(), h_prev_fp8=inp["h_prev_fp8"].numpy(),
        dn_hh_fp8=u8(inp["dn_hh_fp8"]), dn_hh_scale=inp["dn_hh_scale"].numpy(),
        up_hh=inp["up_hh"].numpy(), up_ih=inp["up_ih"].numpy(), bhh=inp["bhh"].numpy(),
        bih=inp["bih"].numpy(), x_down=inp["x_down"].numpy(), c=inp["c"].numpy(),
        h_ref=h_ref.numpy(), c_ref=c_ref.numpy())

    for name, d in out.items():
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **d)
        print(f"wrote {name}.npz  ({os.path.getsize(os.path.join(HERE, name + '.npz'))} B)")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
