"""Sharding of quantized layers over the GPUs of one box (one process per GPU).

Column-parallel layers split the OUTPUT rows of the [N, K] GGUF matrix: rank r uploads the
contiguous row range `shard_rows(N, world, r)` (a contiguous byte range of the raw blocks) and
produces a slice of y; the slices are all-gathered.  Row-parallel layers split K in whole
blocks (`shard_cols`): every rank produces a partial y that is all-reduced.  KV heads are
split per rank with `shard_rows(n_kv_heads, world, r)`.

The reference has no multi-device notion (core/src/commonMain/kotlin/sk/ai/net/Tensor.kt:6-33);
this is new surface.  The collectives go through torch.distributed (NCCL on GPUs, gloo in the
CPU tests); no device-side multicast is used anywhere.
"""
from __future__ import annotations

from typing import Tuple


def shard_rows(n_rows: int, world: int, rank: int) -> Tuple[int, int]:
    """(begin, count) of the rows rank `rank` owns; the first n_rows % world ranks own one more."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank outside the world")
    base, extra = divmod(n_rows, world)
    begin = rank * base + min(rank, extra)
    return begin, base + (1 if rank < extra else 0)


def shard_cols(n_cols: int, block: int, world: int, rank: int) -> Tuple[int, int]:
    """(begin, count) of the columns rank `rank` owns, in whole blocks of `block` columns."""
    if n_cols % block:
        raise ValueError(f"Quantized tensor row size ({n_cols}) is not a multiple of block size ({block})")
    b, c = shard_rows(n_cols // block, world, rank)
    return b * block, c * block


def all_gather_rows(y_local, group=None):
    """Concatenate the per-rank slices y_local [..., rows_r] along the last axis (ranks may own
    different counts).  torch tensors on any device the process group supports."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    n = torch.tensor([y_local.shape[-1]], dtype=torch.int64, device=y_local.device)
    sizes = [torch.zeros_like(n) for _ in range(world)]
    dist.all_gather(sizes, n, group=group)
    sizes = [int(s.item()) for s in sizes]
    mx = max(sizes)
    pad = torch.zeros(y_local.shape[:-1] + (mx,), dtype=y_local.dtype, device=y_local.device)
    pad[..., : y_local.shape[-1]] = y_local
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad, group=group)
    return torch.cat([p[..., :s] for p, s in zip(parts, sizes)], dim=-1)


def all_reduce_partials(y_partial, group=None):
    """Sum of the per-rank partial products of a row-parallel layer (in place)."""
    import torch.distributed as dist
    dist.all_reduce(y_partial, op=dist.ReduceOp.SUM, group=group)
    return y_partial
