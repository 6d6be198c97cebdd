"""Weight layout converters against the reference's pre-shuffle (golden vectors)."""
import numpy as np
import torch

from conftest import load_golden
from gigaslop_b200 import layout


def test_preshuffle_matches_reference_and_inverts():
    g = load_golden("fp8_quant")
    wq = torch.from_numpy(g["wq"])                     # E4M3 bytes of B[K, N]
    shuf = layout.preshuffle_b(wq)
    assert np.array_equal(shuf.numpy(), g["w_shuf"])
    w_nk = layout.unshuffle_b(torch.from_numpy(g["w_shuf"]))
    assert torch.equal(w_nk, wq.t().contiguous())
    f16 = torch.from_numpy(g["w_kn"]).half()
    assert np.array_equal(layout.preshuffle_b(f16).numpy(), g["w_shuf_f16"])
    assert torch.equal(layout.unshuffle_b(torch.from_numpy(g["w_shuf_f16"])), f16.t().contiguous())


def test_split_fc1():
    fc1 = torch.arange(4 * 6).reshape(4, 6)
    gate, up = layout.split_fc1(fc1, 3)
    assert torch.equal(gate, fc1[:, :3].t()) and torch.equal(up, fc1[:, 3:].t())
