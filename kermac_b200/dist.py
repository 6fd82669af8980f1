"""Row sharding of the distance operators over the GPUs of one node.

Every output row n (one point of `b`) is independent of the others, so `cdist` and
`kernel_matvec` shard over n with no exchange during compute: rank r owns a contiguous
slab of rows, needs all of `a` (and `c`) and only its rows of `b`.  One collective,
an all-gather of the slabs, runs at the end when the caller wants the full result on
every rank.  The reference has no multi-GPU code; this module is additive.

One process per GPU, `torch.distributed` initialised by the caller (NCCL for CUDA
tensors; the helpers are backend-agnostic, so Gloo ranks on CPU tensors work too).
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist_

__all__ = ["shard_rows", "slab_sizes", "gather_buffer", "gather_rows_inplace", "gather_rows", "cdist_sharded",
           "kernel_matvec_sharded"]


ROW_ALIGN = 128   # slab boundaries fall on output-tile boundaries (and keep slices 16-byte aligned)


def slab_sizes(n: int, world: int, align: int = 1) -> list:
    """Rows per rank: every rank gets the same slab of whole `align`-row units, except that
    the last non-empty slab is cut where the rows end (trailing ranks may own nothing).
    Equal slabs make the all-gather a single in-place collective whose result needs no copy."""
    if world < 1:
        raise ValueError("world must be >= 1")
    if n < 0:
        raise ValueError("n must be >= 0")
    if align < 1:
        raise ValueError("align must be >= 1")
    units = -(-n // align)
    slab = align * (-(-units // world))
    bounds = [min(n, r * slab) for r in range(world + 1)]
    return [bounds[r + 1] - bounds[r] for r in range(world)]


def shard_rows(n: int, rank: int, world: int, align: int = 1) -> Tuple[int, int]:
    """[start, stop) of the rows rank `rank` owns out of n."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} is outside [0, {world})")
    sizes = slab_sizes(n, world, align)
    start = sum(sizes[:rank])
    return start, start + sizes[rank]


def gather_buffer(n_total: int, tail: tuple, world: int, rank: int, align: int, device, dtype=torch.float32):
    """(buffer, slab): a (world * slab_rows, *tail) buffer and the view of it that rank `rank`
    fills.  After `gather_rows_inplace` the first n_total rows of the buffer are the result."""
    sizes = slab_sizes(n_total, world, align)
    largest = max(sizes) if sizes else 0
    buf = torch.empty((world * largest,) + tuple(tail), dtype=dtype, device=device)
    return buf, buf[rank * largest: rank * largest + sizes[rank]]


def gather_rows_inplace(buf: torch.Tensor, n_total: int, group=None) -> torch.Tensor:
    """In-place all-gather of the equal-size slabs of `buf` (see gather_buffer); returns the
    contiguous view buf[:n_total].  Rows of a short or empty last slab carry padding that is
    exchanged but never read."""
    world = dist_.get_world_size(group)
    if world > 1:
        rank = dist_.get_rank(group)
        largest = buf.size(0) // world
        dist_.all_gather_into_tensor(buf, buf[rank * largest: (rank + 1) * largest], group=group)
    return buf[:n_total]


def gather_rows(local: torch.Tensor, n_total: int, group=None, align: int = 1) -> torch.Tensor:
    """All-gathers row slabs (dim 0) of shape (rows_r, ...) into (n_total, ...).

    `local` must be contiguous and follow `slab_sizes(n_total, world, align)`.  This form
    copies the local slab into the gather buffer; operators that can write their slab in
    place use `gather_buffer` + `gather_rows_inplace` instead.
    """
    world = dist_.get_world_size(group)
    rank = dist_.get_rank(group)
    sizes = slab_sizes(n_total, world, align)
    if local.size(0) != sizes[rank]:
        raise ValueError(f"rank {rank} holds {local.size(0)} rows, expected {sizes[rank]}")
    if not local.is_contiguous():
        raise ValueError("local slab must be contiguous")
    if world == 1:
        return local
    buf, slab = gather_buffer(n_total, tuple(local.shape[1:]), world, rank, align, local.device, local.dtype)
    slab.copy_(local)
    return gather_rows_inplace(buf, n_total, group)


def cdist_sharded(a: torch.Tensor, b: torch.Tensor, p: float = 2.0, skip_epilogue: bool = False,
                  group=None, gather: bool = True, compute: Optional[Callable] = None) -> torch.Tensor:
    """Row-sharded `cdist` for 2-D operands.

    Every rank passes the same `a` (M, K) and `b` (N, K).  Returns distances in storage
    order [n][m]: the full (N, M) tensor when `gather`, else this rank's (rows_r, M) slab.
    `compute(a, b_rows, out=...)` defaults to `kermac_b200.cdist`.
    """
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError("cdist_sharded takes 2-D a and b")
    world = dist_.get_world_size(group) if dist_.is_initialized() else 1
    rank = dist_.get_rank(group) if dist_.is_initialized() else 0
    n_total, m_total = b.size(0), a.size(0)
    start, stop = shard_rows(n_total, rank, world, ROW_ALIGN)
    if gather and world > 1:
        buf, slab = gather_buffer(n_total, (m_total,), world, rank, ROW_ALIGN, a.device)
    else:
        buf, slab = None, torch.empty((stop - start, m_total), dtype=torch.float32, device=a.device)
    if compute is None:
        from .cdist import cdist as _cdist

        def compute(a_, b_, out):
            return _cdist(a_, b_, out=out, p=p, skip_epilogue=skip_epilogue)
    if stop > start:
        # `slab` is [n][m] storage; the operator's out is (M, rows) with m contiguous.
        compute(a, b[start:stop], slab.t())
    if buf is None:
        return slab
    return gather_rows_inplace(buf, n_total, group)


def kernel_matvec_sharded(kernel_descriptor, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor,
                          group=None, gather: bool = True, compute: Optional[Callable] = None,
                          **hyper) -> torch.Tensor:
    """Row-sharded `kernel_matvec` for 2-D operands: y (N, O), or this rank's (rows_r, O) slab."""
    if a.dim() != 2 or b.dim() != 2 or c.dim() != 2:
        raise ValueError("kernel_matvec_sharded takes 2-D a, b and c")
    world = dist_.get_world_size(group) if dist_.is_initialized() else 1
    rank = dist_.get_rank(group) if dist_.is_initialized() else 0
    n_total = b.size(0)
    start, stop = shard_rows(n_total, rank, world, ROW_ALIGN)
    if gather and world > 1:
        buf, slab = gather_buffer(n_total, (c.size(0),), world, rank, ROW_ALIGN, a.device)
    else:
        buf, slab = None, torch.empty((stop - start, c.size(0)), dtype=torch.float32, device=a.device)
    if compute is None:
        from .matvec import kernel_matvec as _matvec

        def compute(a_, b_, c_, out):
            return _matvec(kernel_descriptor, a_, b_, c_, out=out, **hyper)
    if stop > start:
        compute(a, b[start:stop], c, slab)
    if buf is None:
        return slab
    return gather_rows_inplace(buf, n_total, group)
