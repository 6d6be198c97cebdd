"""The LSTM entry point for hosts that cannot allocate device memory (scratch lives in a device array built
into the library) must give the same result as the entry point that takes caller scratch -- on two calls in a
row, because every call reuses the same array and has to clear what must start at zero.

This file sorts last on purpose: a run that stops at the first failure has then already run everything else."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(lib, static, ih, W, s, b, T, B, H, reverse, scratch=None):
    h16 = torch.zeros((T * B, H), dtype=torch.float16, device="cuda")
    h8 = torch.zeros((T * B, H), dtype=torch.uint8, device="cuda")
    cl = torch.zeros((B, H), dtype=torch.float16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    common = (ih.data_ptr(), ih.stride(0), W.data_ptr(), W.stride(0), s.data_ptr(), b.data_ptr(), None, None,
              h16.data_ptr(), h8.data_ptr(), cl.data_ptr(), T, B, H, 1 if reverse else 0)
    if static:
        rc = lib.gsb200_lstm_layer_fp8_static(*common, stream)
    else:
        rc = lib.gsb200_lstm_layer_fp8(*common, scratch.data_ptr(), scratch.numel(), stream)
    assert rc == 0, f"status {rc}"
    torch.cuda.synchronize()
    return h16, h8, cl


def test_static_scratch_entry_point_matches_caller_scratch_twice():
    """Shapes with H > 384 run the cooperative kernel, the one that exchanges h through the scratch and counts steps
    in it: with the static entry point that is the array built into the library, reused by the second call (another
    shape, reversed) with the first call's h bytes and counters still in it.  Same kernel, same inputs: the two entry
    points must agree bit for bit.  The third shape (H = 384) takes the cluster kernel, which needs no scratch."""
    import gigaslop_b200 as g
    lib = g.lib()
    gen = torch.Generator().manual_seed(909)
    for (T, B, H, reverse) in [(6, 256, 512, False), (5, 130, 448, True), (20, 256, 384, False)]:
        W = ((torch.rand(4 * H, H, generator=gen) * 2 - 1) * 44.8).to(torch.float8_e4m3fn).cuda()
        s = (torch.full((4 * H,), 1 / 448.0) * (0.9 + 0.2 * torch.rand(4 * H, generator=gen))).cuda()
        b = (0.05 * torch.randn(4 * H, generator=gen)).cuda()
        ih = (torch.randn(T * B, 4 * H, generator=gen) * 0.5).half().cuda()
        scratch = g.lstm_scratch(B, H, "cuda")
        ref = _run(lib, False, ih, W, s, b, T, B, H, reverse, scratch)
        got = _run(lib, True, ih, W, s, b, T, B, H, reverse)
        for name, a, r in zip(("h fp16", "h e4m3", "c"), got, ref):
            assert torch.equal(a, r), f"{name}: static-scratch and caller-scratch entry points differ (T={T}, B={B}, H={H})"
        assert float(got[0].float().abs().max()) > 0.05, "output is all (near) zero: the layer did not run"
        assert g.device_status()[0] == 0


def test_static_scratch_entry_point_rejects_oversize():
    import gigaslop_b200 as g
    lib = g.lib()
    H, B, T = 384, 640, 2                                  # B beyond the built-in array
    ih = torch.zeros(T * B, 4 * H, dtype=torch.float16, device="cuda")
    W = torch.zeros(4 * H, H, dtype=torch.uint8, device="cuda")
    s = torch.ones(4 * H, device="cuda")
    rc = lib.gsb200_lstm_layer_fp8_static(ih.data_ptr(), ih.stride(0), W.data_ptr(), W.stride(0), s.data_ptr(), None,
                                          None, None, None, None, None, T, B, H, 0, None)
    assert rc == -2
