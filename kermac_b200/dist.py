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
           "OverlappedCdist", "kernel_matvec_sharded", "cdist_grad_sharded"]


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


class OverlappedCdist:
    """Row-sharded `cdist` that moves the result to the other ranks while it is computed.

    Rank r owns the contiguous slab of rows `shard_rows(N, r, world, 128)` of the result
    [n][m].  The slab is computed in `chunks` launches; as soon as a launch is done, its
    rows are pushed into the same rows of every peer's result buffer by peer-to-peer
    copies, which the copy engines carry over NVLink without occupying an SM, while the
    next launch computes.  Only the last chunk's push and one cross-rank barrier are not
    hidden.  (A collective on the SMs cannot overlap here: the distance kernels fill every
    SM's register file, so a communication kernel only gets to run between launches.)

    The result buffer is symmetric memory (`torch.distributed._symmetric_memory`), allocated
    and exchanged once per object and reused by every `run`.  Transports:
      "multicast"  (default on CUDA when the NVSwitch multicast object is available) the kernel
                   itself writes its results to the buffer's multicast address with multimem.st,
                   so the switch delivers every row to all GPUs while the kernel computes: one
                   kernel does the computation and the exchange, each GPU sends its slab once;
      "peer_copy"  finished rows are pushed to each peer by copy engines (world - 1 copies of
                   the slab leave every GPU; at 8 GPUs that takes as long as the computation);
      "collective" one in-place all-gather after the last launch (also the CPU / Gloo path).
    """

    def __init__(self, M: int, N: int, device, group=None, chunks: int = 8, transport: str = "auto"):
        if transport not in ("auto", "multicast", "peer_copy", "collective"):
            raise ValueError("transport must be 'auto', 'multicast', 'peer_copy' or 'collective'")
        device = torch.device(device)
        self.group = group
        self.world = dist_.get_world_size(group) if dist_.is_initialized() else 1
        self.rank = dist_.get_rank(group) if dist_.is_initialized() else 0
        self.M, self.N = M, N
        self.sizes = slab_sizes(N, self.world, ROW_ALIGN)
        self.slab_rows = max(self.sizes) if self.sizes else 0
        self.start = sum(self.sizes[:self.rank])
        self.rows = self.sizes[self.rank]
        self.chunks = max(1, chunks)
        symmetric = device.type == "cuda" and self.world > 1 and transport != "collective"
        shape = (self.world * self.slab_rows, M)
        self._handle, self._peers, self._streams, self._second = None, None, None, None
        self.launch_count = 0              # distance-kernel launches issued by this object so far
        if symmetric:
            import torch.distributed._symmetric_memory as symm_mem
            self.full = symm_mem.empty(shape, dtype=torch.float32, device=device)
            self._handle = symm_mem.rendezvous(self.full, group=dist_.group.WORLD if group is None else group)
            has_multicast = bool(getattr(self._handle, "multicast_ptr", 0))
            if transport == "multicast" and not has_multicast:
                raise RuntimeError("this group has no NVSwitch multicast object for symmetric memory")
            if transport == "auto":
                transport = "multicast" if has_multicast else "peer_copy"
            if transport == "peer_copy":
                self._peers = [self._handle.get_buffer(r, shape, torch.float32) for r in range(self.world)]
                self._streams = [torch.cuda.Stream(device=device) for _ in range(self.world)]
        else:
            if transport in ("multicast", "peer_copy") and self.world > 1:
                raise RuntimeError(f"transport {transport!r} needs CUDA tensors")
            transport = "collective"
            self.full = torch.empty(shape, dtype=torch.float32, device=device)
        self.transport = transport

    def chunk_bounds(self):
        """[(row0, row1)] of the launches inside this rank's slab, on 128-row boundaries."""
        per = ROW_ALIGN * max(1, -(-(-(-self.rows // ROW_ALIGN)) // self.chunks))
        return [(r0, min(self.rows, r0 + per)) for r0 in range(0, self.rows, per)]

    def run(self, a: torch.Tensor, b: torch.Tensor, p: float = 2.0, skip_epilogue: bool = False,
            gather: bool = True, compute: Optional[Callable] = None) -> torch.Tensor:
        """a (M, K) and b (N, K) identical on every rank.  Returns the (N, M) result [n][m],
        complete on every rank when `gather`; otherwise only this rank's rows are valid.
        The returned tensor aliases the object's buffer: the next `run` overwrites it."""
        if a.dim() != 2 or b.dim() != 2 or a.size(0) != self.M or b.size(0) != self.N:
            raise ValueError("operands do not match the shapes this object was built for")
        if compute is None:
            from .cdist import cdist as _cdist

            def compute(a_, b_, out):
                return _cdist(a_, b_, out=out, p=p, skip_epilogue=skip_epilogue)
        if gather and self.world > 1 and self.transport == "multicast":
            return self._run_multicast(a, b, p, skip_epilogue)
        push = gather and self.world > 1 and self.transport == "peer_copy"
        on_cuda = self.full.is_cuda
        main = torch.cuda.current_stream() if on_cuda else None
        if push:
            self._handle.barrier()          # nobody is still reading the buffer a peer is about to fill
        bounds = self.chunk_bounds()
        # Launches alternate between the caller's stream and a second one: they write disjoint
        # rows, so the next launch's thread blocks fill the SMs the previous one's last wave
        # leaves idle instead of waiting for it to drain.
        second = None
        if on_cuda and len(bounds) > 1:
            if self._second is None:
                self._second = torch.cuda.Stream(device=self.full.device)
            second = self._second
            second.wait_stream(main)
        for g, (r0, r1) in enumerate(bounds):
            rows = slice(self.start + r0, self.start + r1)
            stream = second if (second is not None and g % 2 == 1) else main
            if stream is main:
                compute(a, b[rows], self.full[rows].t())
            else:
                with torch.cuda.stream(stream):
                    compute(a, b[rows], self.full[rows].t())
            self.launch_count += 1
            if push:
                done = torch.cuda.Event()
                done.record(stream)
                for r in range(self.world):
                    if r == self.rank:
                        continue
                    copier = self._streams[r]
                    copier.wait_event(done)
                    with torch.cuda.stream(copier):
                        self._peers[r][rows].copy_(self.full[rows], non_blocking=True)
        if second is not None:
            main.wait_stream(second)
        if push:
            for r in range(self.world):
                if r != self.rank:
                    main.wait_stream(self._streams[r])
            self._handle.barrier()          # every rank's pushes into this buffer have landed
        elif gather and self.world > 1:
            gather_rows_inplace(self.full, self.N, self.group)
        return self.full[:self.N]


def _overlapped_run_multicast(self, a, b, p, skip_epilogue):
    """One launch over this rank's slab whose result stores go to the multicast address of the
    symmetric buffer: every GPU's buffer receives the rows while the kernel runs."""
    from . import _native
    from .build_a_kernel import _current_stream_for, _marshal_build
    from .cdist import descriptor_for
    self._handle.barrier()              # nobody is still reading the rows about to be overwritten
    if self.rows > 0:
        rows = slice(self.start, self.start + self.rows)
        descriptor, powers = descriptor_for(p, skip_epilogue)
        args, _, keep = _marshal_build(descriptor, a, b[rows], self.full[rows].t(), powers.get("p"),
                                       powers.get("inner_p"), None, None, None, None, 0, 0)
        args.out = self._handle.multicast_ptr + self.start * self.M * 4
        args.out_multicast = 1
        _native.launch_build(args, _current_stream_for(a.device))
        self.launch_count += 1
        del keep
    self._handle.barrier()              # every rank's kernel, and with it its multicast stores, is complete
    return self.full[:self.N]


OverlappedCdist._run_multicast = _overlapped_run_multicast


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
            # the slab's row 0 is row `start` of the whole problem: move the diagonal with it
            kw = dict(hyper)
            if kw.get("regularization") is not None:
                kw["regularization_offset_y"] = int(kw.get("regularization_offset_y", 0)) + start
            return _matvec(kernel_descriptor, a_, b_, c_, out=out, **kw)
    if stop > start:
        compute(a, b[start:stop], c, slab)
    if buf is None:
        return slab
    return gather_rows_inplace(buf, n_total, group)


GRAD_ROW_ALIGN = 16   # the gradient kernels tile n in multiples of 16


def cdist_grad_sharded(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, d: torch.Tensor, p=2.0,
                       group=None, gather: bool = True, compute: Optional[Callable] = None) -> torch.Tensor:
    """`cdist_grad` sharded over the rows n of `b` (N, K) and `d` (N, M) for 2-D operands.

    Every output slice out[:, n, :] depends on row n of `b` and `d` only, so rank r computes
    out[:, rows_r, :] from all of `a` (K, M) and `c` (O, K) with no exchange; the contracted
    dimension k is never split across ranks (that would need an all-reduce).  Returns the full
    (O, N, M) tensor when `gather` (one all-gather of the slabs, then a concatenation along n),
    else this rank's (O, rows_r, M) slab.  `compute(a, b_rows, c, d_rows, out=...)` defaults to
    `kermac_b200.cdist_grad`.
    """
    if a.dim() != 2 or b.dim() != 2 or c.dim() != 2 or d.dim() != 2:
        raise ValueError("cdist_grad_sharded takes 2-D a, b, c and d")
    world = dist_.get_world_size(group) if dist_.is_initialized() else 1
    rank = dist_.get_rank(group) if dist_.is_initialized() else 0
    n_total, m_total, o_total = b.size(0), a.size(1), c.size(0)
    if d.size(0) != n_total:
        raise ValueError(f"d must have {n_total} rows like b, got {d.size(0)}")
    sizes = slab_sizes(n_total, world, GRAD_ROW_ALIGN)
    start = sum(sizes[:rank])
    stop = start + sizes[rank]
    largest = max(sizes) if sizes else 0
    if compute is None:
        from .cdist_grad import cdist_grad as _grad

        def compute(a_, b_, c_, d_, out):
            return _grad(a_, b_, c_, d_, out=out, p=p)
    if gather and world > 1:
        buf = torch.empty((world, o_total, largest, m_total), dtype=torch.float32, device=a.device)
        slab = buf[rank, :, :sizes[rank]]
    else:
        buf, slab = None, torch.empty((o_total, stop - start, m_total), dtype=torch.float32, device=a.device)
    if stop > start:
        compute(a, b[start:stop], c, d[start:stop], slab)
    if buf is None:
        return slab
    flat = buf.view(world * o_total, largest, m_total)       # concatenation along dim 0, as the collective expects
    dist_.all_gather_into_tensor(flat, flat[rank * o_total:(rank + 1) * o_total], group=group)
    return torch.cat([buf[r, :, :sizes[r]] for r in range(world) if sizes[r] > 0], dim=1)

