"""Run one kernel of the path on seeded synthetic inputs of a benchmark shape and print its CUDA-event time.

    python -m gigaslop_b200.run_shape <op> [--M rows] [--iters n] [--warmup n]

Used for per-kernel timings and as the command behind the ncu summaries in ``profiles/``.  Inputs rotate over
three buffer sets so that no launch finds its inputs in L2.  Ops (shapes of the benchmark configurations):

    ptq_int8 / ptq_fp8           per-token quantiser, [M, 512] fp16           (--K for another width)
    gemm_i8 / gemm_fp8           dequant GEMM N=512 K=512                       (config 1)
    rotary_i8 / rotary_fp8       QKV GEMM + rotary N=1536 K=512                 (config 2)
    ptq_rotary_i8                per-token quantiser fused into the QKV GEMM + rotary, fp16 in (config 2)
    dual_silu_i8 / dual_silu_fp8 SwiGLU dual GEMM N=2048 K=512                  (config 3)
    down_i8 / down_fp8           down-projection N=512 K=2048                   (config 3)
    dual_silu_mxfp8              FP8 SwiGLU emitting MXFP8                      (config 4)
    mx_gemm / mx_dual_silu       block-scaled (kind::mxf8f6f4) GEMMs N=2048 K=512 (config 4)
    mx_down                      block-scaled down-projection N=512 K=2048      (config 4)
    ih_proj                      hoisted LSTM input projection [M,384]x[1536,384] (config 5; M = T*B)
    lstm_layer                   persistent recurrence, B=512 H=384, T = M / 512  (config 5)
    lstm_stack                   the 5-layer stack of config 5 (hoisted projection + recurrence per layer,
                                 alternating direction), T = M / 512
    fac_gemm                     low-rank input projection C=1024 R=128 N=4096
"""
import argparse

import torch

from . import ops
from .lstm import lstm_layer, lstm_scratch, lstm_stack

DEV = "cuda"


def _i8(g, *s):
    return torch.randint(-127, 128, s, generator=g, dtype=torch.int8).to(DEV)


def _f8(g, *s, amp=448.0):
    return ((torch.rand(s, generator=g) * 2 - 1) * amp).to(torch.float8_e4m3fn).to(DEV)


def _scales(g, n):
    return (1e-3 + 9e-3 * torch.rand(n, generator=g)).to(DEV)


def build(op, M, K):
    """Returns (callable taking a buffer-set index, operations per call or None, algorithmic bytes per call)."""
    g = torch.Generator().manual_seed(1234)
    sets = 3
    if op in ("ptq_int8", "ptq_fp8"):
        xs = [torch.randn(M, K, generator=g).half().to(DEV) for _ in range(sets)]
        q = torch.empty(M, K, dtype=torch.int8 if op == "ptq_int8" else torch.float8_e4m3fn, device=DEV)
        s = torch.empty(M, device=DEV)
        if op == "ptq_int8":
            return (lambda i: ops.quantize_tensor(xs[i], out=q, out_scale=s)), None, M * K * 3 + M * 4
        return (lambda i: ops.fp8_quantize_per_token(xs[i], torch_formulation=False, out=q, out_scale=s)), None, M * K * 3 + M * 4
    if op == "ptq_rotary_i8":
        N, K = 1536, 512
        xs = [torch.randn(M, K, generator=g).half().to(DEV) for _ in range(sets)]
        W = _i8(g, N, K)
        sb = _scales(g, N)
        sin, cos = (t.to(DEV) for t in (torch.randn(2048, 32, generator=g), torch.randn(2048, 32, generator=g)))
        outs = [torch.empty(M, N, dtype=torch.float16, device=DEV) for _ in range(sets)]
        return (lambda i: ops.quantize_gemm_i8_rotary(xs[i], W, sb, sin, cos, 8, 64, 64, 2048, out=outs[i])), \
            2.0 * M * N * K, M * K * 2 + N * K + M * N * 2 + 4 * N
    kind8 = _i8 if op.endswith("i8") else _f8
    if op in ("gemm_i8", "gemm_fp8", "down_i8", "down_fp8", "rotary_i8", "rotary_fp8", "ih_proj"):
        N, K = {"gemm": (512, 512), "down": (512, 2048), "rotary": (1536, 512), "ih": (1536, 384)}[op.split("_")[0]]
        if op == "ih_proj":
            kind8 = _f8
        A = [kind8(g, M, K) for _ in range(sets)]
        W = kind8(g, N, K)
        sa, sb = _scales(g, M), _scales(g, N)
        outs = [torch.empty(M, N, dtype=torch.float16, device=DEV) for _ in range(sets)]
        byts = M * K + N * K + M * N * 2 + 4 * (M + N)
        if op.startswith("rotary"):
            sin, cos = (t.to(DEV) for t in (torch.randn(2048, 32, generator=g), torch.randn(2048, 32, generator=g)))
            fn = ops.gemm_i8_rotary if op == "rotary_i8" else ops.gemm_fp8_rotary
            return (lambda i: fn(A[i], W, sa, sb, sin, cos, 8, 64, 64, 2048, out=outs[i])), 2.0 * M * N * K, byts
        fn = ops.gemm_i8 if kind8 is _i8 else ops.gemm_fp8
        return (lambda i: fn(A[i], W, sa, sb, out=outs[i])), 2.0 * M * N * K, byts
    if op in ("dual_silu_i8", "dual_silu_fp8", "dual_silu_mxfp8"):
        N, K = 2048, 512
        if op == "dual_silu_mxfp8":
            kind8 = _f8
        A = [kind8(g, M, K) for _ in range(sets)]
        Wg, Wu = kind8(g, N, K), kind8(g, N, K)
        sa, sg, su = _scales(g, M), _scales(g, N), _scales(g, N)
        if op == "dual_silu_mxfp8":
            o8 = torch.empty(M, N, dtype=torch.float8_e4m3fn, device=DEV)
            os_ = torch.empty(M, N // 32, dtype=torch.uint8, device=DEV)
            return (lambda i: ops.dual_gemm_fp8_silu_mxfp8(A[i], Wg, Wu, sa, sg, su, out=o8, out_scale=os_)), \
                4.0 * M * N * K, M * K + 2 * N * K + M * N + M * N // 32
        outs = [torch.empty(M, N, dtype=torch.float16, device=DEV) for _ in range(sets)]
        fn = ops.dual_gemm_i8_silu if kind8 is _i8 else ops.dual_gemm_fp8_silu
        return (lambda i: fn(A[i], Wg, Wu, sa, sg, su, out=outs[i])), 4.0 * M * N * K, M * K + 2 * N * K + M * N * 2
    if op in ("mx_gemm", "mx_dual_silu", "mx_down"):
        N, K = (512, 2048) if op == "mx_down" else (2048, 512)
        A = [_f8(g, M, K) for _ in range(sets)]
        sfa = ops.mx_scales_to_tiled(torch.randint(120, 128, (M, K // 32), generator=g, dtype=torch.uint8).to(DEV), K)
        Wg, Wu = _f8(g, N, K), _f8(g, N, K)
        sfg = ops.mx_scales_to_tiled(torch.randint(120, 128, (N, K // 32), generator=g, dtype=torch.uint8).to(DEV), K)
        sfu = ops.mx_scales_to_tiled(torch.randint(120, 128, (N, K // 32), generator=g, dtype=torch.uint8).to(DEV), K)
        outs = [torch.empty(M, N, dtype=torch.float16, device=DEV) for _ in range(sets)]
        if op != "mx_dual_silu":
            return (lambda i: ops.gemm_mxfp8(A[i], sfa, Wg, sfg, out=outs[i])), 2.0 * M * N * K, M * K + N * K + M * N * 2
        return (lambda i: ops.dual_gemm_mxfp8_silu(A[i], sfa, Wg, Wu, sfg, sfu, out=outs[i])), 4.0 * M * N * K, \
            M * K + 2 * N * K + M * N * 2
    if op == "lstm_layer":
        B, H = 512, 384
        T = max(1, M // B)
        W = _f8(g, 4 * H, H, amp=44.8)
        s = torch.full((4 * H,), 1 / 448.0, device=DEV)
        b = torch.zeros(4 * H, device=DEV)
        ih = (torch.randn(T * B, 4 * H, generator=g) * 0.5).half().to(DEV)
        scr = lstm_scratch(B, H, DEV)
        return (lambda i: lstm_layer(ih, W, s, T, B, bias=b, scratch=scr)), 2.0 * T * B * 4 * H * H, \
            T * B * 4 * H * 2 + T * B * H * 3
    if op == "lstm_stack":
        B, H, NL = 512, 384, 5
        T = max(1, M // B)
        layers = []
        for _ in range(NL):
            layers.append(dict(W_ih=_f8(g, 4 * H, H, amp=44.8), s_ih=torch.full((4 * H,), 1 / 448.0, device=DEV),
                               b=(0.05 * torch.randn(4 * H, generator=g)).to(DEV),
                               W_hh=_f8(g, 4 * H, H, amp=44.8), s_hh=torch.full((4 * H,), 1 / 448.0, device=DEV)))
        x8 = _f8(g, T * B, H)
        sx = torch.full((T * B,), 1 / 448.0, device=DEV)
        scr = lstm_scratch(B, H, DEV)
        return (lambda i: lstm_stack(x8, sx, layers, T, B, scratch=scr)), NL * 2 * 2.0 * T * B * 4 * H * H, \
            NL * (T * B * H + 2 * T * B * 4 * H * 2 + T * B * H * 3)
    if op == "fac_gemm":
        C, R, N = 1024, 128, 4096
        x = [_f8(g, M, C, amp=100.0) for _ in range(sets)]
        sx = _scales(g, M)
        dn = _f8(g, R, C)
        sdn = torch.tensor([1e-3], device=DEV)
        up = (torch.randn(N, R, generator=g) * 0.1).half().to(DEV)
        bias = (torch.randn(N, generator=g) * 0.05).to(DEV)
        out = torch.empty(M, N, dtype=torch.float16, device=DEV)
        return (lambda i: ops.fp8_factored_gemm(x[i], sx, dn, sdn, up, bias, out=out)), \
            2.0 * M * (C * R + R * N), M * C + M * N * 2
    raise SystemExit(f"unknown op {op!r}")


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("op")
    ap.add_argument("--M", type=int, default=65536)
    ap.add_argument("--K", type=int, default=512)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args()
    fn, flops, byts = build(a.op, a.M, a.K)
    for i in range(a.warmup):
        fn(i % 3)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.iters):
        fn(i % 3)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / max(a.iters, 1) * 1e3
    line = f"{a.op} M={a.M}: {us:.2f} us per call, {byts / us / 1e3:.0f} GB/s algorithmic"
    if flops:
        line += f", {flops / us / 1e6:.0f} T(FL)OPS"
    from ._lib import device_status
    print(line, "status", device_status())


if __name__ == "__main__":
    main()
