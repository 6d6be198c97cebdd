"""Two-stream front end of the quantise + QKV-rotary path for a stream of device-resident batches.

``quantize_tensor`` and ``gemm_i8_rotary`` of ONE batch depend on each other, those of consecutive batches do
not.  Issued on one stream they run strictly one after the other, and every kernel boundary costs the tail of
one kernel (SMs that have run out of work) plus the ramp of the next.  This helper puts the quantiser on a
second stream: the quantiser of batch i+1 becomes eligible together with the GEMM of batch i and runs under
the GEMM's ramp and tail (the GEMM stream has the higher priority, so its CTAs are placed first; a GEMM CTA
fills an SM's register file, so the quantiser's blocks take whatever SMs are not, or no longer, occupied).

Results are those of the two calls made directly: the kernels and their arguments are the same.
"""
import torch

from . import ops

FLAG_OWN_ROW_BLOCKS = 8      # GSB200_FLAG_OWN_ROW_BLOCKS


class QkvRotaryStreamPipeline:
    """``submit(x, out, ...)`` per batch, ``join()`` after the last; int8 activations and scales live in ``depth`` slots.

    ``x`` is ``[M, K]`` fp16 on the device, ``out`` ``[M, N]`` fp16 on the device; neither may be reused before the
    batch has finished (``join()``, or ``depth`` later submits for ``x``).
    """

    def __init__(self, M, K, N, device, depth=3):
        if depth < 3:
            raise ValueError("depth must be at least 3 (a slot is rewritten two batches after its GEMM was queued)")
        self.M, self.K, self.N = M, K, N
        self.dev = torch.device(device)
        self.depth = depth
        self.sq = torch.cuda.Stream(self.dev, priority=0)       # quantiser
        self.sg = torch.cuda.Stream(self.dev, priority=-1)      # GEMM: placed first when both are pending
        self.q = [torch.empty(M, K, dtype=torch.int8, device=self.dev) for _ in range(depth)]
        self.s = [torch.empty(M, dtype=torch.float32, device=self.dev) for _ in range(depth)]
        self.qdone = [torch.cuda.Event() for _ in range(depth)]
        self.gdone = [torch.cuda.Event() for _ in range(depth)]
        self.n = 0

    def submit(self, x, out, w, s_w, sin, cos, nhead, head_dim, rotary_dim, seqlen, row_offset=0, events=None):
        """Queue one batch.  ``events``: optional pair of CUDA events recorded around the GEMM on its stream."""
        if tuple(x.shape) != (self.M, self.K) or tuple(out.shape) != (self.M, self.N):
            raise ValueError("tensor shapes do not match the pipeline")
        cur = torch.cuda.current_stream(self.dev)
        self.sq.wait_stream(cur)
        self.sg.wait_stream(cur)
        n, b = self.n, self.n % self.depth
        with torch.cuda.stream(self.sq):
            if n >= 2:          # eligible together with the GEMM of the batch before; also frees slot b (GEMM n - depth)
                self.sq.wait_event(self.gdone[(n - 2) % self.depth])
            ops.quantize_tensor(x, out=self.q[b], out_scale=self.s[b])
            self.qdone[b].record(self.sq)
        with torch.cuda.stream(self.sg):
            self.sg.wait_event(self.qdone[b])
            if events is not None:
                events[0].record(self.sg)
            # no sharing of the last round's row blocks: the next batch's quantiser is what fills those SMs here
            ops.gemm_i8_rotary(self.q[b], w, self.s[b], s_w, sin, cos, nhead, head_dim, rotary_dim, seqlen,
                               row_offset=row_offset, out=out, flags=FLAG_OWN_ROW_BLOCKS)
            if events is not None:
                events[1].record(self.sg)
            self.gdone[b].record(self.sg)
        self.n += 1

    def join(self):
        """The current stream waits for every batch queued so far (no host synchronisation)."""
        cur = torch.cuda.current_stream(self.dev)
        cur.wait_stream(self.sg)
        cur.wait_stream(self.sq)

    def finish(self):
        """The host waits for every batch queued so far."""
        self.join()
        torch.cuda.current_stream(self.dev).synchronize()


class QkvRotaryGraph:
    """The quantise + QKV-rotary step of a ring of device-resident batches, captured once into a CUDA graph.

    ``capture(xs, outs, ...)`` records ``repeat`` passes over the given batches (one quantiser and one GEMM launch
    per batch, on one stream, in order); ``replay()`` launches them all with one call.  Launched this way the two
    kernels of a step follow each other without the gap an eager launch leaves (83 us per 65536-token step against
    89-97 us for eager launches on one or two streams, B200).  The reference drives its per-step LSTM launches the same
    way (fly/bench_factored_lstm.py:104-121).  Results are those of the direct calls: same kernels, same arguments.

    ``steps`` overrides the number of steps (default ``repeat`` passes over the batches; step i works on batch
    i % len(xs)).  ``time_gemms`` additionally captures a second graph of the same steps with a pair of CUDA events
    around GEMM launches (``replay(timed=True)``; afterwards ``gemm_events[i][0].elapsed_time(gemm_events[i][1])`` is
    the duration of a GEMM inside the step): ``True`` = around every GEMM, an integer n = around n of them, evenly
    spaced.  An event node costs about 4 us, which is why they live in a graph of their own and can be few.
    """

    def __init__(self, M, K, N, device, slots=3):
        self.M, self.K, self.N = M, K, N
        self.dev = torch.device(device)
        self.q = [torch.empty(M, K, dtype=torch.int8, device=self.dev) for _ in range(slots)]
        self.s = [torch.empty(M, dtype=torch.float32, device=self.dev) for _ in range(slots)]
        self.graph = None
        self.timed_graph = None
        self.gemm_events = []
        self.steps = 0

    def capture(self, xs, outs, w, s_w, sin, cos, nhead, head_dim, rotary_dim, seqlen, row_offset=0, repeat=1,
                time_gemms=False, steps=None):
        if len(xs) != len(outs) or len(xs) > len(self.q):
            raise ValueError("one output per batch, and no more batches than slots")
        n_steps = repeat * len(xs) if steps is None else int(steps)
        if n_steps < 1:
            raise ValueError("at least one step")
        n_timed = n_steps if time_gemms is True else min(int(time_gemms), n_steps)
        timed_at = {(k * n_steps) // n_timed + (n_steps // n_timed) // 2 for k in range(n_timed)} if n_timed else set()
        def one(b, ev):
            ops.quantize_tensor(xs[b], out=self.q[b], out_scale=self.s[b])
            if ev is not None:
                ev[0].record()
            ops.gemm_i8_rotary(self.q[b], w, self.s[b], s_w, sin, cos, nhead, head_dim, rotary_dim, seqlen,
                               row_offset=row_offset, out=outs[b])
            if ev is not None:
                ev[1].record()
        with torch.cuda.device(self.dev):
            for b in range(len(xs)):                 # eager once: first-call set-up happens outside the capture
                one(b, None)
            torch.cuda.synchronize()
            self.gemm_events = []
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                for i in range(n_steps):
                    one(i % len(xs), None)
            if n_timed:
                self.timed_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.timed_graph):
                    for i in range(n_steps):
                        ev = None
                        if i in timed_at:
                            ev = (torch.cuda.Event(enable_timing=True, external=True),
                                  torch.cuda.Event(enable_timing=True, external=True))
                            self.gemm_events.append(ev)
                        one(i % len(xs), ev)
            self.steps = n_steps
        return self

    def replay(self, timed=False):
        """Launch every captured step on the current stream (``timed``: the copy with events around the GEMMs)."""
        (self.timed_graph if timed else self.graph).replay()
