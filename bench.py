#!/usr/bin/env python
"""Benchmark of the quantized-GEMM hot path on B200.

Headline workload (benchmark configuration 2): per-token INT8 quantisation of fp16 activations [65536, 512] followed
by the W8A8 QKV GEMM [65536,512]x[1536,512]^T with the rotary embedding fused into the epilogue.  One step = one pass
of that chain over the batch.  With N GPUs every rank owns its own 65536-row batch (weak scaling, rows are
independent, no collective on the data path).

    python bench.py --gpus N --steps K --warmup W          # this library: one JSON line (rank 0)
    python bench.py --impl reference ...                    # the reference's CPU (PyTorch) math, same JSON shape
    python bench.py --only <op> [--M rows] [--iters n]      # one kernel of the path by itself (profiling target)
    python bench.py --role-timers <op> [--M rows]           # where one launch of a GEMM kernel waits, role by role

Beside the headline keys the JSON line carries
    configs            every kernel and chain of the five benchmark configurations: CUDA-event time, T(FL)OPS, GB/s
                       and the fraction of the measured and of the nominal tensor / HBM peaks, tokens/s per chain
    tensor_peak_probe  tcgen05.mma issue-rate probe (kind::i8, kind::f8f6f4; N = 128, 256): the tensor-side peak
                       measured on this GPU
    sustained          the headline step repeated for over a second (clocks and power-cap flag beside it)
    host_us_per_call   host time of one C-ABI call (tensor maps cached) for the per-step entry points
"""
import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the QKV+rotary GEMM at the bench's full size, from an
# ncu capture of this kernel on this workload (35.6 MB read + 141.5 MB written, the mean of two launches)
GEMM_DRAM_TRAFFIC = 177.2e6
WORKLOAD = ("config2: per-token int8 quantise [65536,512] fp16 + W8A8 QKV GEMM N=1536 K=512 "
            "with fused rotary (8 heads x 64, seqlen 2048), per GPU")
METRIC = "w8a8_qkv_rotary_gemm_tops"
UNIT = "TOPS"
NOMINAL_TENSOR_TOPS = 4500.0      # dense INT8 = FP8 tcgen05 peak of a B200 (datasheet)
NOMINAL_HBM_GBS = 8000.0
DEV = "cuda"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler(threading.Thread):
    """Polls SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.stop_flag, self.max_mhz = index, [], set(), False, None
        self.power = []
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def sample(self):
        if not self.ok:
            return
        nv = self.nv
        try:
            self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
            get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
            r = get(self.h)
            names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
            for bit, name in names.items():
                if r & bit:
                    self.reasons.add(name)
            self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
        except Exception:
            pass

    def run(self):
        while not self.stop_flag:
            self.sample()
            time.sleep(0.01)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        out = {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
               "reasons": sorted(self.reasons), "samples": len(self.samples)}
        if self.power:
            out["power_w_max"] = max(self.power)
        return out


# ---------------------------------------------------------------------------------------------------------------------
# CPU arm: the reference's PyTorch math for the step (oracle restatement), all host threads
# ---------------------------------------------------------------------------------------------------------------------
def cpu_chain(x16, w, s_w, sin, cos, cfg):
    """The reference's CPU path for the step: quantize_tensor + rotary_ref (oracle restatement)."""
    import oracle
    q, s = oracle.quantize_tensor(x16.float())
    return oracle.rotary_ref(q, w, s, s_w, sin, cos, cfg["nhead"], cfg["head_dim"], cfg["rotary_dim"], cfg["seqlen"])


def time_cpu(sample_rows, repeats, threads):
    from gigaslop_b200 import inputs
    torch.set_num_threads(threads)
    c = inputs.config2(0, sample_rows)
    cpu_chain(c["x"][:256], c["w"], c["s_w"], c["sin"], c["cos"], c)     # warm
    ts = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        cpu_chain(c["x"], c["w"], c["s_w"], c["sin"], c["cos"], c)
        ts.append(time.perf_counter() - t0)
    return ts, c


def run_reference(args):
    """Reference arm: the reference's CPU (PyTorch fp32) math for the step on all host threads, on the whole 65536-row
    batch per step with the warm-up count asked for.  Only when steps + warm-up of the whole batch would take more than
    about four minutes is the batch cut to a row sample (and the line says so)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from gigaslop_b200 import inputs
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    steps, warm = max(args.steps, 1), max(args.warmup, 0)
    full = inputs.CONFIG2["M"]
    cal, _ = time_cpu(2048, 2, threads)
    est_full = min(cal) * full / 2048.0
    rows = full
    if est_full * (steps + warm) > 240.0:
        rows = int(full * 240.0 / (est_full * (steps + warm)))
        rows = max(128, min(full, rows // 128 * 128))
    c = inputs.config2(0, rows)
    ts = []
    for i in range(steps + warm):
        t0 = time.perf_counter()
        cpu_chain(c["x"], c["w"], c["s_w"], c["sin"], c["cos"], c)
        ts.append(time.perf_counter() - t0)
    ts = ts[warm:]
    sec = sum(ts) / len(ts)
    ops = 2.0 * rows * c["N"] * c["K"]
    val = ops / sec / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "M_per_gpu": full, "N": c["N"], "K": c["K"],
                   "parallelism": "host cores, all threads", "rows_per_step": rows},
        "tokens_per_s": rows / sec,
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{rows} of {full} rows x {steps} steps of config2 (quantize_tensor + rotary_ref, torch CPU fp32)"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------------
# single kernels and chains of the five configurations
# ---------------------------------------------------------------------------------------------------------------------
def _i8(g, *s):
    return torch.randint(-127, 128, s, generator=g, dtype=torch.int8).to(DEV)


def _f8(g, *s, amp=448.0):
    return ((torch.rand(s, generator=g) * 2 - 1) * amp).to(torch.float8_e4m3fn).to(DEV)


def _scales(g, n):
    return (1e-3 + 9e-3 * torch.rand(n, generator=g)).to(DEV)


def _act(dg, m, k):
    return torch.randn(m, k, generator=dg, device=DEV, dtype=torch.float16)


def _i8_dev(dg, m, k):
    return torch.randint(-127, 128, (m, k), generator=dg, device=DEV, dtype=torch.int8)


def _f8_dev(dg, m, k, amp=448.0):
    return ((torch.rand(m, k, generator=dg, device=DEV) * 2 - 1) * amp).to(torch.float8_e4m3fn)


def nsets(bytes_per_set):
    """Buffer sets to rotate over so that a call never finds its operands in the 126 MB L2 (at least three)."""
    return int(max(3, min(16, 280e6 // max(bytes_per_set, 1) + 1)))


OPS = ("ptq_int8", "ptq_fp8", "ptq_mxfp8", "gemm_i8", "gemm_fp8", "rotary_i8", "rotary_fp8", "ptq_rotary_i8",
       "dual_silu_i8", "dual_silu_fp8", "requant_int8", "down_i8", "down_fp8", "dual_silu_mxfp8", "mx_dual_silu",
       "mx_gemm", "mx_down", "ih_proj", "lstm_layer", "lstm_stack", "lstm_stack_overlap", "fac_gemm",
       "factored_lstm_step")


def build_op(op, M, sets=None):
    """(callable taking a call index, operations per call or None, algorithmic bytes per call, bound) for one kernel
    of the path on seeded synthetic inputs of the benchmark's shape.  Inputs and outputs rotate over enough buffer
    sets that no call finds its operands in L2 (``sets`` overrides the count)."""
    import gigaslop_b200 as G
    from gigaslop_b200 import ops
    g = torch.Generator().manual_seed(1234)
    dg = torch.Generator(device=DEV).manual_seed(4321)
    if op in ("ptq_int8", "ptq_fp8", "ptq_mxfp8", "requant_int8"):
        K = 2048 if op == "requant_int8" else 512
        sets = sets or nsets(M * K * 2)
        xs = [_act(dg, M, K) for _ in range(sets)]
        if op == "ptq_mxfp8":
            q = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=DEV)
            s = torch.empty(M, K // 32, dtype=torch.uint8, device=DEV)
            return (lambda i: ops.mxfp8_quantize(xs[i % sets], out=q, out_scale=s)), None, M * K * 3 + M * K // 32, "hbm"
        q = torch.empty(M, K, dtype=torch.int8 if op != "ptq_fp8" else torch.float8_e4m3fn, device=DEV)
        s = torch.empty(M, device=DEV)
        if op == "ptq_fp8":
            return (lambda i: ops.fp8_quantize_per_token(xs[i % sets], torch_formulation=False, out=q, out_scale=s)), None, M * K * 3 + M * 4, "hbm"
        return (lambda i: ops.quantize_tensor(xs[i % sets], out=q, out_scale=s)), None, M * K * 3 + M * 4, "hbm"
    if op == "ptq_rotary_i8":
        N, K = 1536, 512
        sets = sets or nsets(M * K * 2 + M * N * 2)
        xs = [_act(dg, M, K) for _ in range(sets)]
        W, sb = _i8(g, N, K), _scales(g, N)
        sin, cos = (t.to(DEV) for t in (torch.randn(2048, 32, generator=g), torch.randn(2048, 32, generator=g)))
        outs = [torch.empty(M, N, dtype=torch.float16, device=DEV) for _ in range(sets)]
        return (lambda i: ops.quantize_gemm_i8_rotary(xs[i % sets], W, sb, sin, cos, 8, 64, 64, 2048, out=outs[i % sets])), \
            2.0 * M * N * K, M * K * 2 + N * K + M * N * 2 + 4 * N, "hbm"
    kind8 = _i8 if op.endswith("i8") else _f8
    act8 = _i8_dev if op.endswith("i8") else _f8_dev
    if op in ("gemm_i8", "gemm_fp8", "down_i8", "down_fp8", "rotary_i8", "rotary_fp8", "ih_proj"):
        N, K = {"gemm": (512, 512), "down": (512, 2048), "rotary": (1536, 512), "ih": (1536, 384)}[op.split("_")[0]]
        if op == "ih_proj":
            kind8, act8 = _f8, _f8_dev
        sets = sets or (1 if M > 262144 else nsets(M * K + M * N * 2))      # a million rows: one set is 3.5 GB already
        A = [act8(dg, M, K) for _ in range(sets)]
        W = kind8(g, N, K)
        sa, sb = _scales(g, M), _scales(g, N)
        outs = [torch.empty(M, N, dtype=torch.float16, device=DEV) for _ in range(sets)]
        byts = M * K + N * K + M * N * 2 + 4 * (M + N)
        bound = "tensor" if op.startswith("down") else "hbm"
        if op.startswith("rotary"):
            sin, cos = (t.to(DEV) for t in (torch.randn(2048, 32, generator=g), torch.randn(2048, 32, generator=g)))
            fn = ops.gemm_i8_rotary if op == "rotary_i8" else ops.gemm_fp8_rotary
            return (lambda i: fn(A[i % sets], W, sa, sb, sin, cos, 8, 64, 64, 2048, out=outs[i % sets])), 2.0 * M * N * K, \
                byts + 2 * 2048 * 32 * 4, bound
        fn = ops.gemm_i8 if kind8 is _i8 else ops.gemm_fp8
        return (lambda i: fn(A[i % sets], W, sa, sb, out=outs[i % sets])), 2.0 * M * N * K, byts, bound
    if op in ("dual_silu_i8", "dual_silu_fp8", "dual_silu_mxfp8"):
        N, K = 2048, 512
        if op == "dual_silu_mxfp8":
            kind8, act8 = _f8, _f8_dev
        sets = sets or nsets(M * K + M * N * 2)
        A = [act8(dg, M, K) for _ in range(sets)]
        Wg, Wu = kind8(g, N, K), kind8(g, N, K)
        sa, sg, su = _scales(g, M), _scales(g, N), _scales(g, N)
        if op == "dual_silu_mxfp8":
            o8 = torch.empty(M, N, dtype=torch.float8_e4m3fn, device=DEV)
            os_ = torch.empty(M, N // 32, dtype=torch.uint8, device=DEV)
            return (lambda i: ops.dual_gemm_fp8_silu_mxfp8(A[i % sets], Wg, Wu, sa, sg, su, out=o8, out_scale=os_)), \
                4.0 * M * N * K, M * K + 2 * N * K + M * N + M * N // 32, "tensor"
        outs = [torch.empty(M, N, dtype=torch.float16, device=DEV) for _ in range(sets)]
        fn = ops.dual_gemm_i8_silu if kind8 is _i8 else ops.dual_gemm_fp8_silu
        return (lambda i: fn(A[i % sets], Wg, Wu, sa, sg, su, out=outs[i % sets])), 4.0 * M * N * K, M * K + 2 * N * K + M * N * 2, "tensor"
    if op in ("mx_gemm", "mx_dual_silu", "mx_down"):
        N, K = (512, 2048) if op == "mx_down" else (2048, 512)
        sets = sets or nsets(M * K + M * N * 2)
        A = [_f8_dev(dg, M, K) for _ in range(sets)]
        sfa = ops.mx_scales_to_tiled(torch.randint(120, 128, (M, K // 32), generator=g, dtype=torch.uint8).to(DEV), K)
        Wg, Wu = _f8(g, N, K), _f8(g, N, K)
        sfg = ops.mx_scales_to_tiled(torch.randint(120, 128, (N, K // 32), generator=g, dtype=torch.uint8).to(DEV), K)
        sfu = ops.mx_scales_to_tiled(torch.randint(120, 128, (N, K // 32), generator=g, dtype=torch.uint8).to(DEV), K)
        outs = [torch.empty(M, N, dtype=torch.float16, device=DEV) for _ in range(sets)]
        if op != "mx_dual_silu":
            return (lambda i: ops.gemm_mxfp8(A[i % sets], sfa, Wg, sfg, out=outs[i % sets])), 2.0 * M * N * K, \
                M * K + N * K + M * N * 2 + (M + N) * K // 32, "tensor"
        return (lambda i: ops.dual_gemm_mxfp8_silu(A[i % sets], sfa, Wg, Wu, sfg, sfu, out=outs[i % sets])), 4.0 * M * N * K, \
            M * K + 2 * N * K + M * N * 2 + (M + 2 * N) * K // 32, "tensor"
    if op == "lstm_layer":
        B, H = 512, 384
        T = max(1, M // B)
        W = _f8(g, 4 * H, H, amp=44.8)
        s = torch.full((4 * H,), 1 / 448.0, device=DEV)
        b = torch.zeros(4 * H, device=DEV)
        ih = (torch.randn(T * B, 4 * H, generator=dg, device=DEV) * 0.5).half()
        scr = G.lstm_scratch(B, H, DEV)
        from gigaslop_b200.lstm import lstm_layer
        return (lambda i: lstm_layer(ih, W, s, T, B, bias=b, scratch=scr)), 2.0 * T * B * 4 * H * H, \
            T * B * 4 * H * 2 + T * B * H * 3, "latency"
    if op in ("lstm_stack", "lstm_stack_overlap"):
        B, H, NL = 512, 384, 5
        T = max(1, M // B)
        layers = []
        for _ in range(NL):
            layers.append(dict(W_ih=_f8(g, 4 * H, H, amp=44.8), s_ih=torch.full((4 * H,), 1 / 448.0, device=DEV),
                               b=(0.05 * torch.randn(4 * H, generator=g)).to(DEV),
                               W_hh=_f8(g, 4 * H, H, amp=44.8), s_hh=torch.full((4 * H,), 1 / 448.0, device=DEV)))
        x8, sx = ops.fp8_quantize_per_token(_act(dg, T * B, H))
        overlap = op == "lstm_stack_overlap"
        from gigaslop_b200.lstm import lstm_stack, lstm_stack_workspace
        ws = lstm_stack_workspace(T, B, H, DEV, overlap)
        out = torch.empty(T * B, H, dtype=torch.float16, device=DEV)
        aux = torch.cuda.Stream() if overlap else None
        return (lambda i: lstm_stack(x8, sx, layers, T, B, workspace=ws, aux_stream=aux, out=out)), \
            NL * 2 * 2.0 * T * B * 4 * H * H, NL * (T * B * H + 2 * T * B * 4 * H * 2 + T * B * H) + T * B * H * 2, "latency"
    if op == "fac_gemm":
        C, R, N = 1024, 128, 4096
        sets = sets or 3
        x = [_f8_dev(dg, M, C, amp=100.0) for _ in range(sets)]
        sx = _scales(g, M)
        dn = _f8(g, R, C)
        sdn = torch.tensor([1e-3], device=DEV)
        up = (torch.randn(N, R, generator=g) * 0.1).half().to(DEV)
        bias = (torch.randn(N, generator=g) * 0.05).to(DEV)
        out = torch.empty(M, N, dtype=torch.float16, device=DEV)
        return (lambda i: ops.fp8_factored_gemm(x[i % sets], sx, dn, sdn, up, bias, out=out)), \
            2.0 * M * (C * R + R * N), M * C + M * N * 2, "hbm"
    if op == "factored_lstm_step":
        # one timestep of the reference's low-rank cell as its host drives it: recurrent down-projection, then the cell
        # (fly/bench_factored_lstm.py:82-85); B = M rows, H = 1024, K_hh = R = 128 as deployed
        B, H, Kh, R = M, 1024, 128, 128
        h8 = _f8(g, B, H)
        sx = torch.full((B,), 1 / 448.0, device=DEV)
        dn, sdn = _f8(g, Kh, H), torch.tensor([1e-3], device=DEV)
        up_hh = (torch.randn(4 * H, Kh, generator=g) * 0.1).half().to(DEV)
        up_ih = (torch.randn(4 * H, R, generator=g) * 0.1).half().to(DEV)
        bhh, bih = (torch.randn(4 * H, generator=g) * 0.05).to(DEV), (torch.randn(4 * H, generator=g) * 0.05).to(DEV)
        x_down = (torch.randn(B, R, generator=g) * 0.3).half().to(DEV)
        c = torch.zeros(B, H, device=DEV)
        hh_down = torch.empty(B, Kh, dtype=torch.float16, device=DEV)
        hout = torch.empty(B, H, dtype=torch.uint8, device=DEV)

        def step(i):
            ops.fp8_down_proj(h8, sx, dn, sdn, out=hh_down)
            ops.factored_lstm_step(hout, c, hh_down, up_hh, bhh, x_down, up_ih, bih)
        return step, 2.0 * B * (H * Kh + 4 * H * (Kh + R)), B * H + B * H * 4 * 2 + B * H, "latency"
    raise SystemExit(f"unknown op {op!r}; one of {', '.join(OPS)}")


def time_op(fn, iters, warm, graph=True):
    """Microseconds per call: ``iters`` calls after ``warm`` untimed ones, timed with CUDA events on the launching
    stream.  With ``graph`` the timed calls are captured into one CUDA graph and replayed (the warm-up runs eagerly and
    does every first-call set-up): kernels of 5-20 us are otherwise timed at the rate the Python host can launch them.
    The reference times its per-step LSTM launches the same way (fly/bench_factored_lstm.py:104-121)."""
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(warm + i)
        g.replay()                       # once untimed: the first replay uploads the graph
        torch.cuda.synchronize()
        e0.record()
        g.replay()
        e1.record()
    else:
        e0.record()
        for i in range(iters):
            fn(warm + i)
        e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / max(iters, 1) * 1e3


def kernel_record(us, ops_, byts, bound, hbm_peak, tensor_meas):
    r = {"us": round(us, 3), "bound": bound}
    if byts:
        gbs = byts / us / 1e3
        r.update({"gbs": round(gbs, 1), "frac_hbm_measured": round(gbs / hbm_peak, 4), "frac_hbm_nominal": round(gbs / NOMINAL_HBM_GBS, 4)})
    if ops_:
        tops = ops_ / us / 1e6
        r.update({"tops": round(tops, 1), "frac_tensor_nominal": round(tops / NOMINAL_TENSOR_TOPS, 4)})
        if tensor_meas:
            r["frac_tensor_measured"] = round(tops / tensor_meas, 4)
    return r


def run_only(args):
    """One kernel of the path by itself: the command behind the per-kernel profiler captures."""
    import gigaslop_b200 as G
    G.lib()
    torch.cuda.set_device(0)
    M = args.M or {"lstm_layer": 102400, "lstm_stack": 1024000, "lstm_stack_overlap": 1024000, "ih_proj": 1024000,
                   "gemm_i8": 16384, "gemm_fp8": 16384, "ptq_int8": 65536, "fac_gemm": 131072,
                   "factored_lstm_step": 256}.get(args.only, 65536)
    fn, ops_, byts, bound = build_op(args.only, M)
    us = time_op(fn, args.iters, args.warmup if args.warmup < 100 else 5, graph=False)
    line = f"{args.only} M={M}: {us:.2f} us per call, {byts / us / 1e3:.0f} GB/s algorithmic"
    if ops_:
        line += f", {ops_ / us / 1e6:.0f} T(FL)OPS"
    print(line, "status", G.device_status())


ROLE_TIMER_NAMES = ["MMA thread: loop", "MMA thread: waits for accumulator stages", "MMA thread: waits for ring stages",
                    "producer: waits for free ring stages", "producer: loop", "epilogue warp 0 of lane quarter 0: loop",
                    "... waits for accumulators", "... waits for its stores to be read", "... waits for tensor-memory loads",
                    "epilogue warp 1 of lane quarter 0: loop", "... waits for accumulators", "... waits for its stores to be read",
                    "... waits for tensor-memory loads", "MMA thread: waits for the resident operand"]


def run_role_timers(args):
    """Clocks each role of a GEMM kernel spends in its waits, per CTA: builds the library a second time with
    -DGSB200_GEMM_PROF (beside the shipped one; the shipped library carries no timers), runs one launch of the
    kernel in a child process that loads that build, and prints the median / min / max over the CTAs (tensor-memory
    load waits are timed in the rotary epilogues only)."""
    import subprocess
    from gigaslop_b200 import build
    lib = os.path.join(ROOT, "gigaslop_b200", "libgigaslop_b200_prof.so")
    if os.environ.get("GIGASLOP_B200_LIB") != lib:
        build.build(force=True, defines=("GSB200_GEMM_PROF",), out=lib)
        env = dict(os.environ, GIGASLOP_B200_LIB=lib)
        raise SystemExit(subprocess.call([sys.executable, os.path.abspath(__file__), "--role-timers", args.role_timers,
                                          "--M", str(args.M)], env=env))
    import statistics
    import gigaslop_b200 as G
    G.lib()
    torch.cuda.set_device(0)
    fn, _, _, _ = build_op(args.role_timers, args.M or 65536)
    prof = ctypes.CDLL(lib).gsb200_debug_gemm_prof
    buf = (ctypes.c_longlong * (160 * 16))()
    for i in range(6):
        fn(i)
    torch.cuda.synchronize()
    prof(buf)                                        # clears the timers
    fn(0)
    torch.cuda.synchronize()
    prof(buf)
    print(f"{args.role_timers}: clocks per CTA in one launch (median / min / max over the CTAs that reported)")
    for slot, name in enumerate(ROLE_TIMER_NAMES):
        v = [buf[c * 16 + slot] for c in range(160) if buf[c * 16 + slot] > 0]
        if v:
            print(f"  {name:52s} {statistics.median(v):9.0f} {min(v):9.0f} {max(v):9.0f}   ({len(v)} CTAs)")
    print("status", G.device_status())


def tensor_peak_probe(G):
    """tcgen05.mma issue-rate probe: TOPS of back-to-back MMAs that never touch global memory."""
    L = G.lib()
    clocks = torch.zeros(2 * 256, dtype=torch.int64, device=DEV)
    ctas = ctypes.c_int32(0)
    st = torch.cuda.current_stream().cuda_stream
    out = {}
    mmas = 16384
    for kind, kname in ((0, "i8"), (1, "e4m3")):
        for n in (128, 256):
            for rep in range(2):                    # first launch warms the clocks
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                rc = L.gsb200_tensor_peak_probe(kind, n, mmas, clocks.data_ptr(), ctypes.byref(ctas), st)
                e1.record()
                torch.cuda.synchronize()
                if rc != 0:
                    raise RuntimeError(f"tensor peak probe failed: status {rc}")
            ms = e0.elapsed_time(e1)
            c = clocks[: 2 * ctas.value].view(-1, 2).cpu()
            if int(c[:, 1].min()) < 0:
                raise RuntimeError("tensor peak probe: a bounded wait gave up")
            ops_ = 2.0 * 128 * n * 32 * mmas * ctas.value
            out[f"{kname}_n{n}"] = {"tops": round(ops_ / (ms * 1e-3) / 1e12, 1), "ms": round(ms, 4), "ctas": ctas.value,
                                    "mac_per_clk_per_sm": round(128.0 * n * 32 * mmas / float(c[:, 1].double().mean()), 1),
                                    "issue_clk_per_mma": round(float(c[:, 0].double().mean()) / mmas, 1)}
    out["peak_tops"] = max(v["tops"] for v in out.values())
    out["nominal_tops"] = NOMINAL_TENSOR_TOPS
    out["note"] = ("launch time by CUDA events, 16384 MMAs of M=128 per CTA, one CTA per SM; operands in shared memory; "
                   "peak_tops is the tensor-side denominator of frac_tensor_measured")
    return out


def host_us_per_call(G):
    """Wall-clock host time of one C-ABI call once the tensor maps of its buffers are cached: 500 calls queued without
    synchronising (fewer than the launch queue holds), (a) straight through ctypes with prepared pointers, which is what
    a C/C++ host pays plus the ctypes marshalling, and (b) through the torch-facing wrappers of ``gigaslop_b200.ops``."""
    from gigaslop_b200 import ops
    L = G.lib()
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(7)
    out = {}
    # QKV + rotary GEMM on a 128-row problem
    M, N, K = 128, 1536, 512
    A, W = _i8(g, M, K), _i8(g, N, K)
    sa, sb = _scales(g, M), _scales(g, N)
    sin, cos = torch.randn(2048, 32, generator=g).to(DEV), torch.randn(2048, 32, generator=g).to(DEV)
    C_ = torch.empty(M, N, dtype=torch.float16, device=DEV)
    rot_args = (A.data_ptr(), K, W.data_ptr(), K, C_.data_ptr(), N, sa.data_ptr(), sb.data_ptr(), sin.data_ptr(), cos.data_ptr(),
                M, N, K, 8, 64, 64, 2048, 0, 0, st)
    rot_py = lambda: ops.gemm_i8_rotary(A, W, sa, sb, sin, cos, 8, 64, 64, 2048, out=C_)
    # one timestep of the reference's low-rank LSTM cell: recurrent down-projection + cell, B = 256
    B, H, Kh, R = 256, 1024, 128, 128
    h8 = _f8(g, B, H); sx = torch.full((B,), 1 / 448.0, device=DEV)
    dn, sdn = _f8(g, Kh, H), torch.tensor([1e-3], device=DEV)
    up_hh = (torch.randn(4 * H, Kh, generator=g) * 0.1).half().to(DEV)
    up_ih = (torch.randn(4 * H, R, generator=g) * 0.1).half().to(DEV)
    bhh, bih = torch.zeros(4 * H, device=DEV), torch.zeros(4 * H, device=DEV)
    x_down = (torch.randn(B, R, generator=g) * 0.3).half().to(DEV)
    c = torch.zeros(B, H, device=DEV)
    hh_down = torch.empty(B, Kh, dtype=torch.float16, device=DEV)
    hout = torch.empty(B, H, dtype=torch.uint8, device=DEV)
    dp_args = (h8.data_ptr(), H, dn.data_ptr(), H, hh_down.data_ptr(), Kh, sx.data_ptr(), sdn.data_ptr(), B, Kh, H, 4, st)
    cell_args = (hout.data_ptr(), c.data_ptr(), hh_down.data_ptr(), up_hh.data_ptr(), bhh.data_ptr(), x_down.data_ptr(),
                 up_ih.data_ptr(), bih.data_ptr(), B, H, Kh, R, st)

    def step_c():
        L.gsb200_gemm_fp8_f16(*dp_args)
        L.gsb200_factored_lstm_step(*cell_args)

    def step_py():
        ops.fp8_down_proj(h8, sx, dn, sdn, out=hh_down)
        ops.factored_lstm_step(hout, c, hh_down, up_hh, bhh, x_down, up_ih, bih)

    for name, f_c, f_py, calls in (("gsb200_gemm_i8_rotary_f16", lambda: L.gsb200_gemm_i8_rotary_f16(*rot_args), rot_py, 1),
                                   ("gsb200_gemm_fp8_f16 + gsb200_factored_lstm_step (one LSTM timestep)", step_c, step_py, 2)):
        rec = {"c_abi_calls_per_sample": calls}
        for key, f in (("c_abi_us", f_c), ("python_wrapper_us", f_py)):
            for _ in range(20):
                f()
            torch.cuda.synchronize()
            enc0 = int(L.gsb200_tensor_map_encodes())
            n = 400 // calls
            t0 = time.perf_counter()
            for _ in range(n):
                f()
            t1 = time.perf_counter()
            torch.cuda.synchronize()
            rec[key] = round((t1 - t0) / n * 1e6, 2)
            rec["tensor_maps_encoded"] = int(L.gsb200_tensor_map_encodes()) - enc0
        out[name] = rec
    return out


CONFIG_LEGS = {
    # configuration -> list of (record name, op, rows)
    "config1": [("quantize_int8", "ptq_int8", 16384), ("gemm_i8_dequant", "gemm_i8", 16384)],
    "config2": [("quantize_int8", "ptq_int8", 65536), ("qkv_rotary_i8", "rotary_i8", 65536),
                ("fused_quantize_qkv_rotary_i8", "ptq_rotary_i8", 65536)],
    "config3": [("dual_silu_i8", "dual_silu_i8", 65536), ("requantize_int8_2048", "requant_int8", 65536),
                ("down_proj_i8", "down_i8", 65536)],
    "config4": [("quantize_fp8", "ptq_fp8", 65536), ("qkv_rotary_fp8", "rotary_fp8", 65536),
                ("dual_silu_fp8", "dual_silu_fp8", 65536), ("down_proj_fp8", "down_fp8", 65536),
                ("quantize_mxfp8", "ptq_mxfp8", 65536), ("dual_silu_fp8_emit_mxfp8", "dual_silu_mxfp8", 65536),
                ("mx_dual_silu", "mx_dual_silu", 65536), ("mx_down_proj", "mx_down", 65536)],
    "config5": [("ih_proj_fp8", "ih_proj", 1024000), ("lstm_layer_200_steps", "lstm_layer", 102400),
                ("lstm_stack_5_layers", "lstm_stack", 1024000), ("lstm_stack_5_layers_pipelined", "lstm_stack_overlap", 1024000)],
    "reference_lstm_cell": [("factored_lstm_step_B256", "factored_lstm_step", 256),
                            ("factored_input_projection_M131072", "fac_gemm", 131072)],
}
CHAINS = {
    # chain -> (configuration, tokens per pass, member records whose times add up on one stream)
    "config1_quantize_gemm": ("config1", 16384, ["quantize_int8", "gemm_i8_dequant"]),
    "config3_swiglu_ffn": ("config3", 65536, ["dual_silu_i8", "requantize_int8_2048", "down_proj_i8"]),
    "config4_fp8_qkv": ("config4", 65536, ["quantize_fp8", "qkv_rotary_fp8"]),
    "config4_mx_ffn": ("config4", 65536, ["dual_silu_fp8_emit_mxfp8", "mx_down_proj"]),
}


def run_config_legs(hbm_peak, tensor_meas, iters):
    """Every kernel of the five configurations by itself (CUDA events, rotating buffer sets), then the chains."""
    out = {}
    for cfg, legs in CONFIG_LEGS.items():
        out[cfg] = {}
        for name, op, M in legs:
            fn, ops_, byts, bound = build_op(op, M)
            big = op.startswith("lstm") or op == "ih_proj"
            us = time_op(fn, 3 if big else iters, 2 if big else 5, graph=not big)
            rec = kernel_record(us, ops_, byts, bound, hbm_peak, tensor_meas)
            rec["rows"] = M
            if op == "lstm_layer":
                rec["us_per_step"] = round(us / (M // 512), 3)
            if op.startswith("lstm_stack"):
                rec["ms"] = round(us / 1e3, 3)
                rec["tokens_per_s"] = round(M / (us * 1e-6))
            if op == "factored_lstm_step":
                rec["launches_per_step"] = 2
            out[cfg][name] = rec
            del fn
            torch.cuda.empty_cache()
    for cname, (cfg, tokens, members) in CHAINS.items():
        us = sum(out[cfg][m]["us"] for m in members)
        out[cfg][cname] = {"us": round(us, 3), "tokens_per_s": round(tokens / (us * 1e-6)), "members": members,
                           "note": "sum of the members' CUDA-event times (same stream, one after the other)"}
    return out


# ---------------------------------------------------------------------------------------------------------------------
# headline
# ---------------------------------------------------------------------------------------------------------------------
def run_native(args):
    global DEV
    import gigaslop_b200 as g
    from gigaslop_b200 import inputs
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    g.lib()                                          # fail loudly if the CUDA library is missing
    cfg = inputs.config2()
    M, K, N = cfg["M"], cfg["K"], cfg["N"]
    dev = torch.device("cuda", local)
    # weak scaling: each rank processes its own M-row batch; rank r's rows are global rows r*M..(r+1)*M of the job
    x_host = cfg["x"].pin_memory()
    w = cfg["w"].to(dev); s_w = cfg["s_w"].to(dev); sin = cfg["sin"].to(dev); cos = cfg["cos"].to(dev)
    NSETS = 3            # rotate buffer sets (> L2 in total: 3 x 302 MB) so no step re-reads its inputs from L2
    xs = [x_host.to(dev, non_blocking=True).clone() for _ in range(NSETS)]
    outs = [torch.empty(M, N, dtype=torch.float16, device=dev) for _ in range(NSETS)]
    row_offset = rank * M

    # A step = quantise batch b, then the QKV+rotary GEMM on it.  The steps are captured into CUDA graphs, twelve to
    # a replay (four passes over the three buffer sets), so that the two kernels of a step follow each other without
    # the gap an eager launch leaves; every step's two kernels are launched, and finish, inside the timed region.
    # Steps that do not fill a twelve-step replay run from a second, shorter graph.  The last graph launched in the
    # timed region is a copy with CUDA events around three of its GEMMs (an event node costs about 4 us, so not more).
    from gigaslop_b200.devpipe import QkvRotaryGraph
    G = 12
    n_events = 3
    def make_runner(steps, like=None):
        r = QkvRotaryGraph(M, K, N, dev, slots=NSETS)
        if like is not None:
            r.q, r.s = like.q, like.s                    # one set of int8 buffers for all graphs
        return r.capture(xs, outs, w, s_w, sin, cos, cfg["nhead"], cfg["head_dim"], cfg["rotary_dim"], cfg["seqlen"],
                         row_offset=row_offset, steps=steps, time_gemms=n_events)
    runner = make_runner(G)
    rest = make_runner(args.steps % G, like=runner) if args.steps % G else None
    last = rest if rest is not None else runner          # the graph whose timed copy closes the region

    def eager_step(i):
        b = i % NSETS
        g.quantize_tensor(xs[b], out=runner.q[b], out_scale=runner.s[b])
        g.gemm_i8_rotary(runner.q[b], w, runner.s[b], s_w, sin, cos, cfg["nhead"], cfg["head_dim"], cfg["rotary_dim"],
                         cfg["seqlen"], row_offset=row_offset, out=outs[b])

    def run_steps(n, time_last=False):
        reps, tail = n // G, n % G
        for r in range(reps):
            runner.replay(timed=time_last and tail == 0 and r == reps - 1)
        if tail:
            if rest is not None and tail == rest.steps:
                rest.replay(timed=time_last)
            else:
                for i in range(tail):
                    eager_step(i)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    runner.replay(timed=True)                        # every graph uploaded before anything is timed
    runner.replay()
    if rest is not None:
        rest.replay(timed=True)
        rest.replay()
    sampler = ClockSampler(local)                    # (NVML set-up takes milliseconds: before the warm-up, not after it)
    sampler.sample()
    run_steps(args.warmup)
    barrier()                                        # nothing but the two event objects between this and the first launch
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    run_steps(args.steps, time_last=True)
    t1.record()
    # The clock sampler starts once the region's launches are queued (they take the host tens of microseconds, the GPU
    # works on them for milliseconds): its NVML queries go through the same driver as the launches, and a launch held
    # up by a query leaves the GPU idle inside a region this short.  Its samples are taken while the region executes.
    sampler.start()
    barrier()
    sampler.sample()
    sampler.stop_flag = True
    ms_step = max_over_ranks(t0.elapsed_time(t1)) / args.steps
    # duration of GEMM launches inside the timed region: the events captured around three GEMMs of the region's last
    # graph launch
    gemm_ms = [a.elapsed_time(b) for a, b in last.gemm_events]
    st = g.device_status()
    if st[0] != 0:
        raise RuntimeError(f"device status word reports a timed-out wait: {st}")

    # ---- the same step repeated for over a second: what the GPU sustains once power and clocks have settled ----
    sus_sampler = ClockSampler(local)
    sus_sampler.start()
    n_sus = max(20, int(1.2e3 / max(ms_step, 1e-3)) // G) * G
    s0 = torch.cuda.Event(enable_timing=True); s1 = torch.cuda.Event(enable_timing=True)
    s0.record()
    run_steps(n_sus)
    s1.record()
    barrier()
    sus_sampler.sample()
    sus_sampler.stop_flag = True
    sus_ms = max_over_ranks(s0.elapsed_time(s1)) / n_sus

    # ---- the GEMM kernel by itself (nothing beside it on the GPU), for comparison with its time inside the step ----
    # A short burst after a pause: hundreds of GEMMs back to back run into the power cap, which says nothing about
    # the kernel.
    time.sleep(0.3)
    n_alone = 24
    ea = torch.cuda.Event(enable_timing=True); eb = torch.cuda.Event(enable_timing=True)
    for i in range(n_alone + 3):
        if i == 3:
            ea.record()
        b = i % NSETS
        g.gemm_i8_rotary(runner.q[b], w, runner.s[b], s_w, sin, cos, cfg["nhead"], cfg["head_dim"], cfg["rotary_dim"],
                         cfg["seqlen"], row_offset=row_offset, out=outs[b])
    eb.record()
    torch.cuda.synchronize()
    gemm_alone_ms = ea.elapsed_time(eb) / n_alone

    # ---- end to end through the public API with host buffers (H2D + kernels + D2H every step) ----
    # gigaslop_b200.hostpipe cuts the rows into chunks and overlaps upload, compute and download.
    from gigaslop_b200.hostpipe import QkvRotaryHostPipeline
    out_host = torch.empty(M, N, dtype=torch.float16).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))
    pipe = QkvRotaryHostPipeline(M, K, N, dev)

    def e2e_pass(copy_only):
        def one():
            pipe.run(x_host, out_host, w, s_w, sin, cos, cfg["nhead"], cfg["head_dim"], cfg["rotary_dim"],
                     cfg["seqlen"], row_offset=row_offset, join=False, copy_only=copy_only)
        for _ in range(2):
            one()
        pipe.join()
        barrier()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):      # consecutive steps are pipelined: a step's upload overlaps the download tail of the one before
            one()
        pipe.join()                      # the current stream (and e1) waits for the last download
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)) / e2e_steps

    e2e_ms = e2e_pass(False)
    ceiling_ms = e2e_pass(True)          # the same copies on the same streams with no kernel in between

    # ---- every other kernel and chain of the five configurations, the tensor-peak probe, host time per call ----
    hbm_peak, bf16_peak, which = peaks()
    del xs, outs, pipe, out_host, runner
    torch.cuda.empty_cache()
    DEV = f"cuda:{local}"
    probe = tensor_peak_probe(g)
    configs = run_config_legs(hbm_peak, probe["peak_tops"], iters=20)
    if dist is not None:                 # max over ranks of every leg's time (each rank ran its own copy of the work)
        keys = [(c, k) for c in configs for k in configs[c]]
        t = torch.tensor([configs[c][k]["us"] for c, k in keys], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        for (c, k), us in zip(keys, t.tolist()):
            scale = configs[c][k]["us"] / us if us > 0 else 1.0
            for f in ("gbs", "tops", "frac_hbm_measured", "frac_hbm_nominal", "frac_tensor_nominal", "frac_tensor_measured", "tokens_per_s"):
                if f in configs[c][k]:
                    configs[c][k][f] = round(configs[c][k][f] * scale * (world if f in ("tokens_per_s",) else 1), 4)
            configs[c][k]["us"] = round(us, 3)
    host_us = host_us_per_call(g) if rank == 0 else None
    st = g.device_status()
    if st[0] != 0:
        raise RuntimeError(f"device status word reports a timed-out wait: {st}")

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    ops_step = 2.0 * M * N * K
    value = world * ops_step / (ms_step * 1e-3) / 1e12
    # algorithmic bytes of one QKV+rotary launch: int8 A + int8 W + fp16 C + scales + sin/cos tables
    gemm_bytes = M * K + N * K + M * N * 2 + M * 4 + N * 4 + 2 * cfg["seqlen"] * 32 * 4
    gemm_avg_ms = sum(gemm_ms) / len(gemm_ms)
    achieved = gemm_bytes / (gemm_avg_ms * 1e-3) / 1e9
    gemm_tops = ops_step / (gemm_avg_ms * 1e-3) / 1e12
    cpu_rows = 8192
    cpu_sec = None
    if world == 1:                   # the CPU baseline is reported at N=1 only
        cpu_ts, _ = time_cpu(cpu_rows, 4, os.cpu_count() or 1)
        cpu_sec = min(cpu_ts)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "M_per_gpu": M, "N": N, "K": K, "parallelism": f"row-sharded x{world}, no collective",
                   "l2": f"{NSETS} rotating buffer sets of 302 MB (> 126 MB L2)",
                   "launch": "devpipe.QkvRotaryGraph: the steps are captured into a CUDA graph (12 steps per replay, the steps left over from a shorter graph; one stream) and replayed"},
        "tokens_per_s": world * M / (ms_step * 1e-3),
        "kernel_tops": {"qkv_rotary_gemm": gemm_tops,
                        "frac_of_nominal_4500": gemm_tops / NOMINAL_TENSOR_TOPS,
                        "frac_of_probe_peak": gemm_tops / probe["peak_tops"],
                        "frac_of_2x_bf16_" + which: gemm_tops / (2 * bf16_peak),
                        "step_minus_gemm_ms": ms_step - gemm_avg_ms, "gemm_ms": gemm_avg_ms},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                     "frac": achieved / hbm_peak, "traffic": GEMM_DRAM_TRAFFIC, "peak_source": which,
                     "frac_of_nominal_8000": achieved / NOMINAL_HBM_GBS,
                     "kernel": "gemm_tcgen05_kernel<i8, rotary, activation-stationary, CTA pairs, 12 epilogue warps>", "bytes_per_launch": gemm_bytes,
                     "timed": "CUDA events captured in the step graph around GEMM launches, on the launching stream: %d launches of the timed region's last graph launch" % len(gemm_ms),
                     "achieved_alone": gemm_bytes / (gemm_alone_ms * 1e-3) / 1e9,
                     "frac_alone": gemm_bytes / (gemm_alone_ms * 1e-3) / 1e9 / hbm_peak},
        "e2e": {"value": world * ops_step / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
                "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2, "ms_per_step": e2e_ms,
                "copy_ceiling_ms": ceiling_ms, "frac_of_copy_ceiling": ceiling_ms / e2e_ms,
                "copy_ceiling_note": "the same H2D / D2H copies through the same three streams with no kernel launched",
                "api": "gigaslop_b200.hostpipe.QkvRotaryHostPipeline.run(join=False) + join() (pinned host buffers, 8192-row chunks on 3 streams, consecutive steps pipelined)"},
        "sustained": {"steps": n_sus, "ms_per_step": sus_ms, "value": world * ops_step / (sus_ms * 1e-3) / 1e12, "unit": UNIT,
                      "seconds": sus_ms * n_sus / 1e3, "clocks": sus_sampler.summary()},
        "gpu_launches": 2 * args.steps,
        "clocks": sampler.summary(),
        "tensor_peak_probe": probe,
        "configs": configs,
        "host_us_per_call": host_us,
    }
    if cpu_sec is not None:
        line["cpu_baseline"] = {"value": 2.0 * cpu_rows * N * K / cpu_sec / 1e12, "unit": UNIT,
                                "cores": os.cpu_count() or 1, "kind": "port",
                                "sample": f"{cpu_rows} of 65536 rows, best of 4 (quantize_tensor + rotary_ref, torch CPU fp32)"}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=400)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--only", default=None, help="time one kernel of the path by itself: " + ", ".join(OPS))
    ap.add_argument("--M", type=int, default=0, help="rows for --only")
    ap.add_argument("--iters", type=int, default=20, help="timed calls for --only")
    ap.add_argument("--role-timers", default=None, metavar="OP",
                    help="per-role wait clocks of one launch of a GEMM kernel (builds a profiling copy of the library)")
    args = ap.parse_args()
    if args.role_timers:
        run_role_timers(args)
    elif args.only:
        run_only(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
