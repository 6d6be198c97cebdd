"""Row (token) sharding of the hot path across GPUs.

Every row of the quantiser and of every GEMM epilogue is independent, so the
multi-GPU form of the path is a contiguous split of M with replicated weights
and no collective on the data path; rotary keeps global positions through the
``row_offset`` argument.  ``gather_rows`` is the single optional final exchange.
"""
import torch


def shard_rows(M, world_size, rank, granule=1):
    """Contiguous shard ``[start, start+rows)`` of ``M`` rows for ``rank``.

    Rows are dealt in units of ``granule`` (e.g. one chunk of ``seqlen`` steps, or a 128-row
    tile); the first ``extra`` ranks get one more unit, the tail unit may be ragged."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError("bad world_size / rank")
    units = (M + granule - 1) // granule
    base, extra = divmod(units, world_size)
    u0 = rank * base + min(rank, extra)
    u1 = u0 + base + (1 if rank < extra else 0)
    start = min(u0 * granule, M)
    stop = min(u1 * granule, M)
    return start, stop - start


def gather_rows(local, M, world_size, granule=1, group=None):
    """All-gather row shards produced with :func:`shard_rows` back into ``[M, ...]`` on every rank.
    The only collective of the path; it is outside the kernels and outside kernel timing."""
    import torch.distributed as dist
    if world_size == 1:
        return local
    sizes = [shard_rows(M, world_size, r, granule)[1] for r in range(world_size)]
    mx = max(sizes)
    pad = torch.zeros((mx,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]] = local
    outs = [torch.empty_like(pad) for _ in range(world_size)]
    dist.all_gather(outs, pad, group=group)
    return torch.cat([o[:n] for o, n in zip(outs, sizes)], dim=0)
