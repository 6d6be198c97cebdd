"""Host-buffer front end of the quantise + QKV-rotary path.

The C ABI (like the reference's ``cute_dsl_*_wrapper`` / ``fp8_*_wrapper`` entry
points) takes device pointers.  A caller whose activations and results live in
host memory pays PCIe for both directions; this helper hides what can be hidden:
the rows are cut into chunks and three streams (upload, compute, download) work
on different chunks at the same time, so a step costs about the slower of the
two copy directions instead of their sum.

Results are identical to one whole-batch call: the quantiser and the GEMM are
row-wise, and each chunk's first row goes to the rotary kernel as ``row_offset``.

Back-to-back batches: ``run(..., join=False)`` leaves the three streams running, so
the upload and the kernels of the next batch overlap the download tail of this one
(the device-side slots are handed on through events across calls); ``join()`` makes
the current stream wait for everything queued so far, ``finish()`` the host.
"""
import torch

from . import ops


class QkvRotaryHostPipeline:
    """Reusable pipeline for ``[M, K]`` fp16 host activations -> ``[M, N]`` fp16 host QKV.

    ``x_host`` and ``out_host`` must be pinned.  Weights, scales and tables stay on the device.
    """

    def __init__(self, M, K, N, device, chunk_rows=8192, depth=4):
        self.M, self.K, self.N = M, K, N
        self.dev = torch.device(device)
        self.chunk = min(chunk_rows, M)
        self.depth = depth
        self.h2d = torch.cuda.Stream(self.dev)
        self.cmp = torch.cuda.Stream(self.dev)
        self.d2h = torch.cuda.Stream(self.dev)
        c = self.chunk
        self.x = [torch.empty(c, K, dtype=torch.float16, device=self.dev) for _ in range(depth)]
        self.q = [torch.empty(c, K, dtype=torch.int8, device=self.dev) for _ in range(depth)]
        self.s = [torch.empty(c, dtype=torch.float32, device=self.dev) for _ in range(depth)]
        self.o = [torch.empty(c, N, dtype=torch.float16, device=self.dev) for _ in range(depth)]
        self.up = [torch.cuda.Event() for _ in range(depth)]      # chunk uploaded
        self.done = [torch.cuda.Event() for _ in range(depth)]    # chunk computed
        self.free_x = [torch.cuda.Event() for _ in range(depth)]  # x slot consumed by the quantiser
        self.free_o = [torch.cuda.Event() for _ in range(depth)]  # o slot downloaded
        self.issued = 0                                           # chunks queued since construction (slot = issued % depth)

    def run(self, x_host, out_host, w, s_w, sin, cos, nhead, head_dim, rotary_dim, seqlen, row_offset=0, join=True,
            copy_only=False):
        """Enqueue one pass over all rows; returns after the work is queued.  ``finish()`` waits for it.

        ``join=True`` makes the current stream wait for the pass; with ``join=False`` the caller calls ``join()``
        (or ``finish()``) after the last of a series of passes, and may not touch ``out_host`` before that.
        ``copy_only=True`` queues the same copies with the same dependencies but launches no kernel (``out_host`` then
        receives whatever the device slots hold): the time of such a pass is the ceiling the host link sets.
        """
        if not (x_host.is_pinned() and out_host.is_pinned()):
            raise ValueError("host buffers must be pinned (page-locked) for asynchronous copies")
        if tuple(x_host.shape) != (self.M, self.K) or tuple(out_host.shape) != (self.M, self.N):
            raise ValueError("host buffer shapes do not match the pipeline")
        cur = torch.cuda.current_stream(self.dev)
        for st in (self.h2d, self.cmp, self.d2h):
            st.wait_stream(cur)
        n_chunks = (self.M + self.chunk - 1) // self.chunk
        for i in range(n_chunks):
            b = self.issued % self.depth
            reuse = self.issued >= self.depth                 # the slot has been used before, in this pass or an earlier one
            self.issued += 1
            r0 = i * self.chunk
            rows = min(self.chunk, self.M - r0)
            with torch.cuda.stream(self.h2d):
                if reuse:
                    self.h2d.wait_event(self.free_x[b])
                self.x[b][:rows].copy_(x_host[r0:r0 + rows], non_blocking=True)
                self.up[b].record(self.h2d)
            with torch.cuda.stream(self.cmp):
                self.cmp.wait_event(self.up[b])
                if reuse:
                    self.cmp.wait_event(self.free_o[b])
                if not copy_only:
                    ops.quantize_tensor(self.x[b][:rows], out=self.q[b][:rows], out_scale=self.s[b][:rows])
                self.free_x[b].record(self.cmp)
                if not copy_only:
                    ops.gemm_i8_rotary(self.q[b][:rows], w, self.s[b][:rows], s_w, sin, cos, nhead, head_dim,
                                       rotary_dim, seqlen, row_offset=row_offset + r0, out=self.o[b][:rows])
                self.done[b].record(self.cmp)
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_event(self.done[b])
                out_host[r0:r0 + rows].copy_(self.o[b][:rows], non_blocking=True)
                self.free_o[b].record(self.d2h)
        if join:
            self.join()

    def join(self):
        """The current stream waits for every pass queued so far (no host synchronisation)."""
        cur = torch.cuda.current_stream(self.dev)
        cur.wait_stream(self.d2h)
        cur.wait_stream(self.cmp)
        cur.wait_stream(self.h2d)

    def finish(self):
        """The host waits for every pass queued so far."""
        self.join()
        torch.cuda.current_stream(self.dev).synchronize()
