"""Host side of the LSTM stack: per layer, the hoisted input projection (an FP8 GEMM over all T*B rows) and
the persistent recurrent kernel; layers alternate direction and feed each other E4M3 ``h`` at scale 1/448."""
import torch

from ._lib import check, lib
from .ops import _on_device, _stream

OUT_SCALE = 1.0 / 448.0


def lstm_scratch(B, H, device):
    """Scratch buffer (h exchange + step counters) for :func:`lstm_layer`; reusable across layers and calls
    that do not overlap on the device."""
    n = int(lib().gsb200_lstm_scratch_bytes(B, H))
    return torch.empty(n, dtype=torch.uint8, device=device)


@_on_device
def lstm_layer(ih, W_hh, s_hh, T, B, bias=None, reverse=False, h0=None, c0=None, scratch=None,
               want_h16=True, want_h8=True, want_c=False):
    """Recurrent half of one layer.  ``ih`` fp16 ``[T*B, 4H]`` (row = t*B + b), ``W_hh`` E4M3 ``[4H, H]``.
    Returns (h16 ``[T*B,H]`` or None, h8 ``[T*B,H]`` or None, c_last ``[B,H]`` or None)."""
    H = W_hh.shape[1]
    dev = ih.device
    if scratch is None:
        scratch = lstm_scratch(B, H, dev)
    h16 = torch.empty((T * B, H), dtype=torch.float16, device=dev) if want_h16 else None
    h8 = torch.empty((T * B, H), dtype=torch.float8_e4m3fn, device=dev) if want_h8 else None
    c_last = torch.empty((B, H), dtype=torch.float16, device=dev) if want_c else None
    ptr = lambda t: t.data_ptr() if t is not None else None
    check(lib().gsb200_lstm_layer_fp8(ih.data_ptr(), ih.stride(0), W_hh.data_ptr(), W_hh.stride(0), s_hh.data_ptr(),
                                      ptr(bias), ptr(h0), ptr(c0), ptr(h16), ptr(h8), ptr(c_last), T, B, H,
                                      1 if reverse else 0, scratch.data_ptr(), scratch.numel(), _stream(ih)), "lstm_layer")
    return h16, h8, c_last


def lstm_stack_workspace(T, B, H, device, overlap=False):
    """Workspace of :func:`lstm_stack` (hoisted projections, E4M3 hand-over buffers, layer scratch)."""
    n = int(lib().gsb200_lstm_stack_workspace_bytes(T, B, H, 1 if overlap else 0))
    return torch.empty(n, dtype=torch.uint8, device=device)


def lstm_stack(x_fp8, sx, layers, T, B, reverse_first=True, workspace=None, aux_stream=None, time_blocks=0, out=None):
    """Stack of layers (dicts with W_ih, s_ih, b, W_hh, s_hh); even layers run reversed when ``reverse_first``.
    ``x_fp8`` E4M3 ``[T*B, C]`` with per-row scales ``sx``.  Returns the last layer's fp16 ``h`` ``[T*B, H]``.
    One call into the library (``gsb200_lstm_stack_fp8``).  With ``aux_stream`` (a ``torch.cuda.Stream``) the next
    layer's hoisted projection runs per time block beside the recurrence of the current layer; same bytes."""
    from ._lib import LstmLayer
    H = layers[0]["W_hh"].shape[1]
    C = x_fp8.shape[1]
    dev = x_fp8.device
    overlap = aux_stream is not None and len(layers) > 1
    if workspace is None:
        workspace = lstm_stack_workspace(T, B, H, dev, overlap)
    arr = (LstmLayer * len(layers))()
    for i, L in enumerate(layers):
        arr[i].w_ih, arr[i].ld_w_ih, arr[i].s_ih = L["W_ih"].data_ptr(), L["W_ih"].stride(0), L["s_ih"].data_ptr()
        arr[i].w_hh, arr[i].ld_w_hh, arr[i].s_hh = L["W_hh"].data_ptr(), L["W_hh"].stride(0), L["s_hh"].data_ptr()
        arr[i].bias = L["b"].data_ptr() if L.get("b") is not None else None
    h16 = out if out is not None else torch.empty((T * B, H), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        check(lib().gsb200_lstm_stack_fp8(x_fp8.data_ptr(), x_fp8.stride(0), sx.data_ptr(), C, arr, len(layers),
                                          1 if reverse_first else 0, h16.data_ptr(), T, B, H, time_blocks,
                                          workspace.data_ptr(), workspace.numel(), _stream(x_fp8),
                                          aux_stream.cuda_stream if overlap else None), "lstm_stack")
    return h16


@_on_device
def lstm_layer_static(ih, W_hh, s_hh, T, B, bias=None, reverse=False, h0=None, c0=None,
                      want_h16=True, want_h8=True, want_c=False):
    """:func:`lstm_layer` for hosts that must not allocate device memory inside the library call: the kernel's
    scratch comes from a device array built into the library (B <= 512, H <= 512).  The output tensors are still
    the caller's; pass preallocated ones through the C ABI directly if torch's allocator is off limits too.
    Calls on one device share that array and must not overlap."""
    H = W_hh.shape[1]
    dev = ih.device
    h16 = torch.empty((T * B, H), dtype=torch.float16, device=dev) if want_h16 else None
    h8 = torch.empty((T * B, H), dtype=torch.float8_e4m3fn, device=dev) if want_h8 else None
    c_last = torch.empty((B, H), dtype=torch.float16, device=dev) if want_c else None
    ptr = lambda t: t.data_ptr() if t is not None else None
    check(lib().gsb200_lstm_layer_fp8_static(ih.data_ptr(), ih.stride(0), W_hh.data_ptr(), W_hh.stride(0),
                                             s_hh.data_ptr(), ptr(bias), ptr(h0), ptr(c0), ptr(h16), ptr(h8),
                                             ptr(c_last), T, B, H, 1 if reverse else 0, _stream(ih)), "lstm_layer_static")
    return h16, h8, c_last
