"""Sharding of quantized layers over the GPUs of one box (one process per GPU).

Column-parallel layers split the OUTPUT rows of the [N, K] GGUF matrix: rank r uploads the
contiguous row range `shard_rows(N, world, r)` (a contiguous byte range of the raw blocks) and
produces a slice of y; the slices are all-gathered.  Row-parallel layers split K in whole
blocks (`shard_cols`): every rank produces a partial y that is all-reduced.  KV heads are
split per rank with `shard_rows(n_kv_heads, world, r)`.

The reference has no multi-device notion (core/src/commonMain/kotlin/sk/ai/net/Tensor.kt:6-33);
this is new surface.  Two routes: `Exchange` (skn_comm_*: the library's own push kernels over
peer memory, what the tensor-parallel decoder uses) and the torch.distributed helpers at the end
(NCCL on GPUs, gloo in the CPU tests).  No device-side multicast is used anywhere.
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


class Exchange:
    """One rank's end of the library's inter-GPU exchange (skn_comm_*).

    `Exchange.connect_processes(ctx, capacity, group)`: one process per GPU; the inter-process
    handles travel through torch.distributed (any backend: they are host bytes).
    `Exchange.connect_local([ctx0, ctx1, ...], capacity)`: one process driving several GPUs."""

    def __init__(self, ctx, rank: int, world: int, capacity_floats: int):
        import ctypes
        from . import _ffi
        from .tensor import _check
        self.ctx, self.rank, self.world = ctx, rank, world
        self._h = ctypes.c_void_p()
        _check(ctx.handle, _ffi.lib().skn_comm_create(ctx.handle, rank, world, capacity_floats, ctypes.byref(self._h)))

    @property
    def handle(self):
        return self._h

    def ipc_handle(self) -> bytes:
        import ctypes
        from . import _ffi
        from .tensor import _check
        buf = ctypes.create_string_buffer(_ffi.lib().skn_comm_handle_bytes())
        _check(self.ctx.handle, _ffi.lib().skn_comm_handle(self._h, buf))
        return buf.raw

    @classmethod
    def connect_processes(cls, ctx, capacity_floats: int, group=None) -> "Exchange":
        import torch.distributed as dist
        from . import _ffi
        from .tensor import _check
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        ex = cls(ctx, rank, world, capacity_floats)
        if world > 1:
            blobs = [None] * world
            dist.all_gather_object(blobs, ex.ipc_handle(), group=group)
            _check(ctx.handle, _ffi.lib().skn_comm_connect(ex._h, b"".join(blobs)))
            dist.barrier(group=group)      # nobody pushes before every inbox is mapped
        return ex

    @classmethod
    def connect_local(cls, ctxs, capacity_floats: int):
        import ctypes
        from . import _ffi
        from .tensor import _check
        exs = [cls(c, r, len(ctxs), capacity_floats) for r, c in enumerate(ctxs)]
        arr = (ctypes.c_void_p * len(exs))(*[e._h.value for e in exs])
        try:
            _check(ctxs[0].handle, _ffi.lib().skn_comm_connect_local(arr, len(exs)))
        except Exception:
            for e in exs:
                e.close()
            raise
        return exs

    def all_reduce(self, partial_dev, resid_dev, out_dev, n: int):
        """out = resid + sum over ranks of partial (device pointers or torch tensors)."""
        from . import _ffi
        from .tensor import _check
        ptr = lambda t: None if t is None else (t.data_ptr() if hasattr(t, "data_ptr") else t)
        _check(self.ctx.handle, _ffi.lib().skn_allreduce_dev(self._h, ptr(partial_dev), ptr(resid_dev), ptr(out_dev), n))

    def close(self):
        import ctypes
        from . import _ffi
        if self._h:
            _ffi.lib().skn_comm_destroy(self._h)
            self._h = ctypes.c_void_p()


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
