#!/usr/bin/env python
"""Benchmark of the quantized-GEMM hot path on B200.

Workload (BASELINE config 2): per-token INT8 quantisation of fp16 activations
[65536, 512] followed by the W8A8 QKV GEMM [65536,512]x[1536,512]^T with the rotary
embedding fused into the epilogue.  One step = one pass of that chain over the
batch.  With N GPUs every rank owns its own 65536-row batch (weak scaling, rows
are independent, no collective on the data path).

    python bench.py --gpus N --steps K --warmup W          # this library
    python bench.py --impl reference ...                    # the reference's CPU (PyTorch) math

Prints one JSON line (rank 0).
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the QKV+rotary GEMM at the bench's full size,
# from the ncu capture summarised in profiles/gemm_i8_rotary_config2.md (40.8 MB + 141.6 MB)
GEMM_DRAM_TRAFFIC = 182.4e6
WORKLOAD = ("config2: per-token int8 quantise [65536,512] fp16 + W8A8 QKV GEMM N=1536 K=512 "
            "with fused rotary (8 heads x 64, seqlen 2048), per GPU")
METRIC = "w8a8_qkv_rotary_gemm_tops"
UNIT = "TOPS"


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
        except Exception:
            pass

    def run(self):
        while not self.stop_flag:
            self.sample()
            time.sleep(0.01)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


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
    """Reference arm: the reference's CPU (PyTorch fp32) math for the step on all host threads.
    Each step processes a sample of the 65536 rows sized so that steps+warmup finish in about 90 s."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from gigaslop_b200 import inputs
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    steps, warm = max(args.steps, 1), max(min(args.warmup, 3), 1)
    cal, _ = time_cpu(1024, 2, threads)
    rows = int(1024 * (90.0 / (steps + warm)) / min(cal))
    rows = max(128, min(16384, rows // 128 * 128))
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
        "config": {"workload": WORKLOAD, "M_per_gpu": 65536, "N": c["N"], "K": c["K"],
                   "parallelism": "host cores, all threads", "rows_per_step": rows},
        "tokens_per_s": rows / sec,
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{rows} rows x {steps} steps of config2 (quantize_tensor + rotary_ref, torch CPU fp32)"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_native(args):
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
    qs = [torch.empty(M, K, dtype=torch.int8, device=dev) for _ in range(NSETS)]
    ss = [torch.empty(M, dtype=torch.float32, device=dev) for _ in range(NSETS)]
    outs = [torch.empty(M, N, dtype=torch.float16, device=dev) for _ in range(NSETS)]
    row_offset = rank * M

    # A step = quantise batch b, then the QKV+rotary GEMM on it.  Steps are queued through the package's two-stream
    # pipeline: the quantiser of step i+1 runs on a second stream under the ramp and tail of the GEMM of step i
    # (every step's two kernels are launched, and finish, inside the timed region).
    from gigaslop_b200.devpipe import QkvRotaryStreamPipeline
    spipe = QkvRotaryStreamPipeline(M, K, N, dev, depth=NSETS)
    del qs, ss                                       # the pipeline owns the int8 activations and scales

    def step(i, events=None):
        b = i % NSETS
        spipe.submit(xs[b], outs[b], w, s_w, sin, cos, cfg["nhead"], cfg["head_dim"], cfg["rotary_dim"],
                     cfg["seqlen"], row_offset=row_offset, events=events)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    spipe.join()
    barrier()
    sampler = ClockSampler(local)
    sampler.sample()
    sampler.start()
    n_ev = min(args.steps, 512)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_ev)]
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(args.steps):
        step(i, evs[i] if i < n_ev else None)
    spipe.join()                                     # the timing stream (and t1) waits for the last GEMM
    t1.record()
    barrier()
    sampler.sample()
    sampler.stop_flag = True
    ms_total = t0.elapsed_time(t1)
    gemm_ms = [a.elapsed_time(b) for a, b in evs]
    tt = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms_total = float(tt.item())
    ms_step = ms_total / args.steps
    st = g.device_status()
    if st[0] != 0:
        raise RuntimeError(f"device status word reports a timed-out wait: {st}")

    # ---- the GEMM kernel by itself (nothing beside it on the GPU), for comparison with its time inside the step ----
    # A short burst after a pause: 200 GEMMs back to back run into the power cap (87 us per launch at lowered
    # clocks), which says nothing about the kernel.
    import time
    time.sleep(0.3)
    n_alone = 24
    ea = torch.cuda.Event(enable_timing=True); eb = torch.cuda.Event(enable_timing=True)
    for i in range(n_alone + 3):
        if i == 3:
            ea.record()
        b = i % NSETS
        g.gemm_i8_rotary(spipe.q[b], w, spipe.s[b], s_w, sin, cos, cfg["nhead"], cfg["head_dim"], cfg["rotary_dim"],
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

    def e2e_step():
        pipe.run(x_host, out_host, w, s_w, sin, cos, cfg["nhead"], cfg["head_dim"], cfg["rotary_dim"],
                 cfg["seqlen"], row_offset=row_offset, join=False)

    for _ in range(2):
        e2e_step()
    pipe.join()
    barrier()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):      # consecutive steps are pipelined: a step's upload overlaps the download tail of the one before
        e2e_step()
    pipe.join()                      # the current stream (and e1) waits for the last download
    e1.record()
    barrier()
    te = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te.item()) / e2e_steps

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    ops_step = 2.0 * M * N * K
    value = world * ops_step / (ms_step * 1e-3) / 1e12
    hbm_peak, bf16_peak, which = peaks()
    # algorithmic bytes of one QKV+rotary launch: int8 A + int8 W + fp16 C + scales + sin/cos tables
    gemm_bytes = M * K + N * K + M * N * 2 + M * 4 + N * 4 + 2 * cfg["seqlen"] * 32 * 4
    gemm_avg_ms = sum(gemm_ms) / len(gemm_ms)
    achieved = gemm_bytes / (gemm_avg_ms * 1e-3) / 1e9
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
                   "streams": "devpipe.QkvRotaryStreamPipeline: quantiser of step i+1 on a second stream beside the GEMM of step i"},
        "tokens_per_s": world * M / (ms_step * 1e-3),
        "kernel_tops": {"qkv_rotary_gemm": ops_step / (gemm_avg_ms * 1e-3) / 1e12,
                        "frac_of_2x_bf16_" + which: ops_step / (gemm_avg_ms * 1e-3) / 1e12 / (2 * bf16_peak),
                        "step_minus_gemm_ms": ms_step - gemm_avg_ms, "gemm_ms": gemm_avg_ms},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                     "frac": achieved / hbm_peak, "traffic": GEMM_DRAM_TRAFFIC, "peak_source": which,
                     "kernel": "gemm_tcgen05_kernel<i8, rotary>", "bytes_per_launch": gemm_bytes,
                     "timed": "CUDA events around each GEMM launch of the timed region, on the GEMM's stream, the next step's quantiser running beside it",
                     "achieved_alone": gemm_bytes / (gemm_alone_ms * 1e-3) / 1e9,
                     "frac_alone": gemm_bytes / (gemm_alone_ms * 1e-3) / 1e9 / hbm_peak},
        "e2e": {"value": world * ops_step / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
                "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2, "ms_per_step": e2e_ms,
                "api": "gigaslop_b200.hostpipe.QkvRotaryHostPipeline.run(join=False) + join() (pinned host buffers, 8192-row chunks on 3 streams, consecutive steps pipelined)"},
        "gpu_launches": 2 * args.steps,
        "clocks": sampler.summary(),
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
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
