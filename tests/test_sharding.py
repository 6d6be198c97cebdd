"""Host logic of the multi-GPU form of the path: contiguous row shards, and that
processing shards independently (with the rotary row offset) reproduces the
unsharded result bit for bit.  The 2-rank case runs as gloo processes on CPU with
the oracle standing in for the device kernels."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from gigaslop_b200.sharding import gather_rows, shard_rows


def test_shards_partition_rows():
    for M, g in [(65536, 2048), (1000, 128), (5, 1), (1024000, 2000)]:
        for w in (1, 2, 3, 4, 8):
            parts = [shard_rows(M, w, r, g) for r in range(w)]
            assert parts[0][0] == 0 and sum(n for _, n in parts) == M
            for (s0, n0), (s1, _) in zip(parts, parts[1:]):
                assert s0 + n0 == s1
            assert all(s % g == 0 for s, n in parts if n)


def _case():
    gen = torch.Generator().manual_seed(21)
    M, K, nhead, hd, seqlen = 96, 64, 1, 64, 16
    N = 3 * nhead * hd
    x = torch.randn(M, K, generator=gen)
    B = torch.randint(-127, 128, (N, K), generator=gen, dtype=torch.int8)
    sb = 1e-3 + 9e-3 * torch.rand(N, generator=gen)
    sin, cos = oracle.rope_tables(seqlen, 32, hd)
    return x, B, sb, sin, cos, (nhead, hd, 64, seqlen)


def _shard_result(x, B, sb, sin, cos, dims, start, rows):
    q, s = oracle.quantize_tensor(x[start:start + rows])
    pad = start % dims[3]
    qp = torch.cat([torch.zeros(pad, q.shape[1], dtype=torch.int8), q])
    sp = torch.cat([torch.ones(pad), s])
    return oracle.rotary_exact(qp, B, sp, sb, sin, cos, *dims)[pad:]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, B, sb, sin, cos, dims = _case()
    start, rows = shard_rows(x.shape[0], world, rank, granule=8)
    local = _shard_result(x, B, sb, sin, cos, dims, start, rows)
    full = gather_rows(local.float(), x.shape[0], world, granule=8)
    if rank == 0:
        ret["full"] = full.clone()
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_equals_single(tmp_path):
    x, B, sb, sin, cos, dims = _case()
    whole = _shard_result(x, B, sb, sin, cos, dims, 0, x.shape[0]).float()
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert torch.equal(ret["full"], whole)
