"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no dataset is involved: the reference itself benchmarks
on ``torch.randn`` activations, cute/bench_gemm_i8_rotary.py:34-38).

One generator per tensor, seed = 1000*config + tensor index, generated on CPU so
every rank and the CPU baseline see identical values."""
import torch


def _gen(cfg, idx):
    return torch.Generator().manual_seed(1000 * cfg + idx)


def channel_scales(cfg, idx, n):
    return 1e-3 + 9e-3 * torch.rand(n, generator=_gen(cfg, idx))


def int8_weight(cfg, idx, n, k):
    return torch.randint(-127, 128, (n, k), generator=_gen(cfg, idx), dtype=torch.int8)


def e4m3_weight(cfg, idx, n, k, amp=448.0):
    w = (torch.rand(n, k, generator=_gen(cfg, idx)) * 2 - 1) * amp
    return w.to(torch.float8_e4m3fn)


def activations(cfg, idx, m, k, row_start=0, rows=None):
    """fp16 N(0,1) activations; a shard regenerates only its rows (row-seeded in blocks of 4096)."""
    rows = m if rows is None else rows
    out = torch.empty(rows, k, dtype=torch.float16)
    blk = 4096
    r = row_start
    while r < row_start + rows:
        b = r // blk
        g = torch.Generator().manual_seed((1000 * cfg + idx) * 100003 + b)
        block = torch.randn(blk, k, generator=g).half()
        lo = r - b * blk
        hi = min(blk, row_start + rows - b * blk)
        out[r - row_start: r - row_start + (hi - lo)] = block[lo:hi]
        r += hi - lo
    return out


def rope_tables(seqlen, rotary_half=32, head_dim=64, base=10000.0):
    inv_freq = 1.0 / (base ** (torch.arange(0, rotary_half).float() / head_dim * 2))
    freqs = torch.outer(torch.arange(seqlen).float(), inv_freq)
    return freqs.sin().contiguous(), freqs.cos().contiguous()


CONFIG2 = dict(M=65536, K=512, N=1536, nhead=8, head_dim=64, rotary_dim=64, seqlen=2048, chunks=32)


def config2(row_start=0, rows=None):
    """QKV projection with fused rotary, INT8: 32 chunks x 2048 steps, d_model 512, W [1536,512]."""
    c = CONFIG2
    sin, cos = rope_tables(c["seqlen"])
    return dict(x=activations(2, 0, c["M"], c["K"], row_start, rows), w=int8_weight(2, 1, c["N"], c["K"]),
                s_w=channel_scales(2, 2, c["N"]), sin=sin, cos=cos, **c)
