"""Oracle: factored (low-rank) projections and LSTM cells (CPU, PyTorch).

Test infrastructure only.

* ``factored_gemm_ref`` / ``down_proj_ref`` / ``factored_lstm_step_ref`` restate
  the reference's own host references (pinned by golden vectors).
* ``lstm_fullrank_*`` is the full-rank sigmoid/tanh cell of the 5-layer
  benchmark stack.  The reference has no such cell (its LSTM is low-rank with
  hard gates), so this part is **parity unpinned**; it mirrors the rounding
  points of the device kernel (E4M3 ``h`` at fixed scale 1/448 feeding the
  recurrent GEMM, fp16 ``h``/``c`` state, fp16 hoisted input projection).
"""
import torch

OUT_SCALE = 1.0 / 448.0


def factored_gemm_ref(x_rows, dn, up, bias):
    """``ih = (x @ dn^T) @ up^T + bias``.  Follows ``fly/bench_factored_gemm.py:54-55``
    (dn ``[R,C]``, up ``[N,R]``, bias ``[N]``, all fp32)."""
    return (x_rows @ dn.t()) @ up.t() + bias


def down_proj_ref(x_fp8, scale_x, dn_fp8_rc, scale_dn):
    """``x_down = (x_fp8 . dn_fp8^T) * sx[m] * s_dn`` in fp32 (dn given ``[R,C]``).
    Follows the epilogue at ``fly/rdna_fp8_factored_gemm.py:486-633`` and the
    host check ``fly/bench_factored_lstm.py:93-94``."""
    acc = x_fp8.float() @ dn_fp8_rc.float().t()
    return acc * scale_x[:, None] * scale_dn.reshape(())


def factored_lstm_step_ref(h_prev_q, dn_hh_fp8, dn_hh_scale, up_hh, x_down, up_ih, bhh, bih, c):
    """One low-rank LSTM step with hard gates.  Follows ``reference()`` at
    ``fly/bench_factored_lstm.py:62-73``: gate order i,f,g,o in blocks of H;
    ``i,f,o = clamp(0.2x+0.5,0,1)``, ``g = clamp(x,-1,1)``, ``c' = f*c + i*g``,
    ``h = o*tanh(c')``.  Returns (h fp32, c' fp32)."""
    dn_hh_dq = dn_hh_fp8.float() * dn_hh_scale.item()
    hh_down = h_prev_q @ dn_hh_dq.t()
    gates = hh_down @ up_hh.t() + x_down.float() @ up_ih.t() + bhh + bih
    i, f, g, o = gates.chunk(4, dim=1)
    i = (i * 0.2 + 0.5).clamp(0, 1)
    f = (f * 0.2 + 0.5).clamp(0, 1)
    g = g.clamp(-1, 1)
    o = (o * 0.2 + 0.5).clamp(0, 1)
    c_new = f * c + i * g
    return o * c_new.tanh(), c_new


def rational_tanh(c):
    """The device approximation of tanh used by the reference kernel
    (``fly/rdna_fp8_factored_lstm.py:315-319``): ``clamp(c(27+c^2)/(27+9c^2), -1, 1)``."""
    x2 = c * c
    return (c * (27.0 + x2) / (27.0 + 9.0 * x2)).clamp(-1, 1)


# ---------------------------------------------------------------------------
# Full-rank cell (benchmark stack).  parity unpinned.
# ---------------------------------------------------------------------------
def _q_h(h):
    """h in [-1,1] -> E4M3 at the fixed scale 1/448 (reference convention,
    ``fly/rdna_fp8_factored_lstm.py:321-326``)."""
    return (h.float() * 448.0).clamp(-448, 448).to(torch.float8_e4m3fn)


def lstm_fullrank_step_ref(ih_t, h_fp8, c, W_hh_fp8, s_hh, bias=None):
    """One step.  ``ih_t`` fp16 ``[B,4H]`` (hoisted input projection incl. bias),
    ``h_fp8`` E4M3 ``[B,H]`` at scale 1/448, ``c`` fp16 ``[B,H]``,
    ``W_hh_fp8`` E4M3 ``[4H,H]`` with per-channel fp32 scales ``s_hh[4H]``.
    gates = ih + (h_fp8 . W^T) * (1/448 * s_hh[n]);  i,f,o sigmoid; g tanh.
    Returns (h fp16, h E4M3, c fp16)."""
    acc = (h_fp8.double() @ W_hh_fp8.double().t()).float()
    gates = ih_t.float() + acc * (OUT_SCALE * s_hh)[None, :]
    if bias is not None:
        gates = gates + bias
    i, f, g, o = gates.chunk(4, dim=1)
    i = torch.sigmoid(i)
    f = torch.sigmoid(f)
    g = torch.tanh(g)
    o = torch.sigmoid(o)
    c_new = f * c.float() + i * g
    h_new = o * torch.tanh(c_new)
    return h_new.to(torch.float16), _q_h(h_new), c_new.to(torch.float16)


def lstm_fullrank_recurrent_ref(ih, W_hh_fp8, s_hh, bias, T, B, reverse, h0_fp8=None, c0=None):
    """T steps over a given hoisted projection ``ih`` fp16 ``[T*B, 4H]`` (row = t*B + b).
    Returns (h fp16 ``[T*B,H]``, its E4M3 image, final c fp16)."""
    H = W_hh_fp8.shape[1]
    h8 = h0_fp8 if h0_fp8 is not None else torch.zeros(B, H).to(torch.float8_e4m3fn)
    c = c0 if c0 is not None else torch.zeros(B, H, dtype=torch.float16)
    out16 = torch.empty(T * B, H, dtype=torch.float16)
    out8 = torch.empty(T * B, H, dtype=torch.float8_e4m3fn)
    order = range(T - 1, -1, -1) if reverse else range(T)
    for t in order:
        h16, h8, c = lstm_fullrank_step_ref(ih[t * B:(t + 1) * B], h8, c, W_hh_fp8, s_hh, bias)
        out16[t * B:(t + 1) * B] = h16
        out8[t * B:(t + 1) * B] = h8
    return out16, out8, c


def lstm_fullrank_layer_ref(x_fp8, sx, W_ih_fp8, s_ih, b, W_hh_fp8, s_hh, reverse, T, B):
    """One layer over T steps.  ``x_fp8`` E4M3 ``[T*B, C]`` with per-row scale ``sx[T*B]`` (row = t*B + b);
    hoisted projection ``(acc * sx) * s_ih`` rounded to fp16 like the device GEMM output; the bias is added
    inside the recurrence.  Returns h fp16 ``[T*B,H]``, its E4M3 image and the final c."""
    acc = (x_fp8.double() @ W_ih_fp8.double().t()).float()
    ih = (acc * sx[:, None] * s_ih[None, :]).to(torch.float16)
    return lstm_fullrank_recurrent_ref(ih, W_hh_fp8, s_hh, b, T, B, reverse)


def lstm_fullrank_stack_ref(x_fp8, sx, layers, T, B, reverse_first=True):
    """Stack of layers with alternating direction; layer l>0 consumes the
    previous layer's E4M3 ``h`` (scale 1/448 for every row)."""
    h16 = None
    for li, L in enumerate(layers):
        rev = (li % 2 == 0) == reverse_first
        h16, h8, _ = lstm_fullrank_layer_ref(x_fp8, sx, L["W_ih"], L["s_ih"], L["b"],
                                             L["W_hh"], L["s_hh"], rev, T, B)
        x_fp8, sx = h8, torch.full((T * B,), OUT_SCALE)
    return h16
