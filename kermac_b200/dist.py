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

__all__ = ["shard_rows", "slab_sizes", "tile_ranges", "tile_coords", "gather_buffer", "gather_rows_inplace", "gather_rows", "cdist_sharded",
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
    """Row-sharded `cdist` for 2-D operands (bit-identical to the single-GPU result for p = 1 and
    p = 2; to rounding for fractional p when a row lands at another position of its tile).

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


def tile_ranges(total: int, world: int) -> list:
    """[(first, count)] per rank: `total` work units in contiguous runs that differ by at most one."""
    if world < 1:
        raise ValueError("world must be >= 1")
    if total < 0:
        raise ValueError("total must be >= 0")
    base, extra = divmod(total, world)
    out, first = [], 0
    for r in range(world):
        count = base + (1 if r < extra else 0)
        out.append((first, count))
        first += count
    return out


TILE = 128          # edge of an output tile of the build kernels
TILE_PANEL = 16     # tile columns (n) per raster panel of the launcher's tile order


def tile_coords(t: int, tiles_m: int, tiles_n: int, panel: int = TILE_PANEL) -> Tuple[int, int]:
    """(tile_m, tile_n) of position t in the build launcher's linear tile order: panels of `panel`
    tile columns, each walked row by row.  Host mirror of the device function of the same name
    (kermac_b200/csrc/km_build_params.cuh), for callers that want to know which part of the output
    a tile range covers."""
    per_panel = panel * tiles_m
    pidx, r = divmod(t, per_panel)
    n0 = pidx * panel
    width = min(panel, tiles_n - n0)
    tm, rest = divmod(r, width)
    return tm, n0 + rest


class OverlappedCdist:
    """Sharded `cdist` that moves the result to the other ranks while it is computed.

    Transports:
      "multicast"  (default on CUDA when the NVSwitch multicast object is available) the kernel
                   itself writes its results to the result buffer's multicast address with
                   multimem.st, so the switch delivers every value to all GPUs while the kernel
                   computes: one kernel does the computation and the exchange, and each GPU sends
                   its share once.  Because such a store can target any element, the work is not
                   cut into row slabs here: the 128 x 128 output tiles are dealt out in equal
                   contiguous runs of the launcher's tile order (`tile_ranges`), which balances
                   the ranks to within one tile whatever N is.  Two result buffers alternate, so a
                   run needs a single cross-rank barrier, at its end: the buffer it writes was
                   last read two runs ago, and every rank has passed a barrier since.
      "peer_copy"  rank r owns the contiguous slab of rows `shard_rows(N, r, world, 128)`; the
                   slab is computed in `chunks` launches and finished rows are pushed to each peer
                   by copy engines while the next launch computes (world - 1 copies of the slab
                   leave every GPU; at 8 GPUs that takes as long as the computation);
      "collective" same slabs, one in-place all-gather after the last launch (also the CPU /
                   Gloo path).  (A collective on the SMs cannot overlap with the computation: the
                   distance kernels fill every SM's register file.)

    The result buffers are symmetric memory (`torch.distributed._symmetric_memory`), allocated
    and exchanged once per object and reused by every `run`.

    A sharded result is bit-identical to the single-GPU one for p = 1 and p = 2: every element
    is the same sequential sum over k wherever its tile runs.  For fractional p it is equal to
    rounding only when the rows land at different positions of a tile (the two exp2 routes).

    None of the launches checks the device error flag: callers poll
    `kermac_b200._native.device_error_flag()` on every rank at their own synchronisation points
    (a bounded wait that ran out leaves the affected tiles unwritten on every rank).
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
        self._buffers, self._handles, self._turn = [], [], 0
        self.launch_count = 0              # distance-kernel launches issued by this object so far
        if symmetric:
            import torch.distributed._symmetric_memory as symm_mem
            grp = dist_.group.WORLD if group is None else group
            self.full = symm_mem.empty(shape, dtype=torch.float32, device=device)
            self._handle = symm_mem.rendezvous(self.full, group=grp)
            has_multicast = bool(getattr(self._handle, "multicast_ptr", 0))
            if transport == "multicast" and not has_multicast:
                raise RuntimeError("this group has no NVSwitch multicast object for symmetric memory")
            if transport == "auto":
                transport = "multicast" if has_multicast else "peer_copy"
            if transport == "peer_copy":
                self._peers = [self._handle.get_buffer(r, shape, torch.float32) for r in range(self.world)]
                self._streams = [torch.cuda.Stream(device=device) for _ in range(self.world)]
            else:
                second = symm_mem.empty(shape, dtype=torch.float32, device=device)
                self._buffers = [self.full, second]
                self._handles = [self._handle, symm_mem.rendezvous(second, group=grp)]
        else:
            if transport in ("multicast", "peer_copy") and self.world > 1:
                raise RuntimeError(f"transport {transport!r} needs CUDA tensors")
            transport = "collective"
            self.full = torch.empty(shape, dtype=torch.float32, device=device)
        self.transport = transport
        self.partition = "tiles" if transport == "multicast" else "rows"
        tiles = (-(-M // 128)) * (-(-N // 128))
        self.tile_first, self.tile_count = tile_ranges(tiles, self.world)[self.rank]
        self._tiles = tiles

    def work_share(self) -> float:
        """Fraction of the whole problem's arithmetic this rank performs."""
        if self.partition == "tiles":
            return self.tile_count / self._tiles if self._tiles else 0.0
        return self.rows / self.N if self.N else 0.0

    def release(self):
        """Drops the result buffers (the object cannot run afterwards)."""
        self.full, self._buffers, self._handles, self._handle, self._peers = None, [], [], None, None

    def chunk_bounds(self):
        """[(row0, row1)] of the launches inside this rank's slab, on 128-row boundaries."""
        per = ROW_ALIGN * max(1, -(-(-(-self.rows // ROW_ALIGN)) // self.chunks))
        return [(r0, min(self.rows, r0 + per)) for r0 in range(0, self.rows, per)]

    def run(self, a: torch.Tensor, b: torch.Tensor, p: float = 2.0, skip_epilogue: bool = False,
            gather: bool = True, compute: Optional[Callable] = None) -> torch.Tensor:
        """a (M, K) and b (N, K) identical on every rank.  Returns the (N, M) result [n][m],
        complete on every rank when `gather`; otherwise only this rank's share is valid.
        The returned tensor aliases one of the object's buffers: with the multicast transport
        the next-but-one `run` overwrites it, with the others the next one.  Like a collective,
        every rank of the group has to make the same sequence of `run` calls with the same
        `gather` flag: the exchange ends in a cross-rank barrier."""
        if a.dim() != 2 or b.dim() != 2 or a.size(0) != self.M or b.size(0) != self.N:
            raise ValueError("operands do not match the shapes this object was built for")
        if self.full is None:
            raise RuntimeError("this object's buffers were released")
        if compute is None:
            from .cdist import cdist as _cdist

            def compute(a_, b_, out):
                return _cdist(a_, b_, out=out, p=p, skip_epilogue=skip_epilogue)
        if self.world > 1 and self.transport == "multicast":
            return self._run_tiles(a, b, p, skip_epilogue, gather)
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

    def _run_tiles(self, a, b, p, skip_epilogue, gather):
        """One launch over this rank's run of output tiles of the WHOLE problem.  With `gather`
        the stores go to the multicast address of the result buffer, so every GPU's buffer
        receives the tiles while the kernel runs; without it they go to this GPU's buffer only."""
        from . import _native
        from .build_a_kernel import _current_stream_for, _marshal_build
        from .cdist import descriptor_for
        turn = self._turn
        buf, handle = self._buffers[turn], self._handles[turn]
        out = buf[:self.N]
        if self.tile_count > 0:
            descriptor, powers = descriptor_for(p, skip_epilogue)
            args, _, keep = _marshal_build(descriptor, a, b, out.t(), powers.get("p"),
                                           powers.get("inner_p"), None, None, None, None, 0, 0)
            if gather:
                args.out = handle.multicast_ptr
                args.out_multicast = 1
            if _native.build_tile_count(args) != self._tiles:
                raise RuntimeError("the launcher's tile count differs from the one the ranks were dealt")
            args.tile_first, args.tile_count = self.tile_first, self.tile_count
            _native.launch_build(args, _current_stream_for(a.device))
            self.launch_count += 1
            del keep
        if gather:
            handle.barrier()            # every rank's kernel, and with it its multicast stores, is complete
            self._turn = 1 - turn       # the next run writes the other buffer: no barrier needed before it
        return out


def kernel_matvec_sharded(kernel_descriptor, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor,
                          group=None, gather: bool = True, compute: Optional[Callable] = None,
                          **hyper) -> torch.Tensor:
    """Row-sharded `kernel_matvec` for 2-D operands: y (N, O), or this rank's (rows_r, O) slab.

    Bit-identical to the single-GPU result as long as the launcher does not split the sum over m
    (small M, or many row tiles); where it does, the split follows the number of thread blocks,
    which sharding changes, and the two results agree to rounding (a few 1e-7 of the largest
    entry).  Pass `split_m` explicitly to pin the grouping."""
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

    Bit-identical to the single-GPU result while the launcher keeps the whole k range in one thread
    block; once it splits k (few output tiles, long K) the split follows the number of thread
    blocks, which sharding changes, and the results agree to rounding only.
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

