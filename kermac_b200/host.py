"""`cdist` for operands and results that live in host memory.

The kermac API takes device tensors (src/kermac/cdist.py:9-83 of the reference); a caller
whose data sits in host memory pays a host-to-device copy of a and b and a device-to-host
copy of the (much larger) distance matrix around it.  `HostCdist` keeps device buffers and
streams for one problem shape and overlaps the three phases: the output rows are cut into
slabs; `a` goes up first, the columns of `b` a slab needs follow slab by slab (strided copies
straight out of the storage layout, no staging), and while slab i is computed, slab i-1 drains
to the host.  The device-to-host copy of the result is the long pole (3.6 GB at the headline
size), so everything else is arranged to let it start as early as possible and never stall.
Nothing here changes what is computed: each slab is a plain `cdist` call.
"""
from __future__ import annotations

import torch

from . import _native
from .cdist import cdist
from .dist import slab_sizes

__all__ = ["HostCdist"]


class HostCdist:
    """Pipelined host-to-host cdist for a[K, M], b[K, N] -> out[N, M] (storage layouts).

    Host tensors should be pinned, otherwise the copies do not overlap.  `slabs` is the
    number of row slabs of the output; two slab buffers rotate on the device.  Computing a slab
    takes about as long as draining it, so equal slabs keep the device-to-host copy busy from the
    first slab on; slabs that grow (to start the drain early and still run large launches) starve
    it, because each takes longer to compute than the previous one takes to drain (measured: 76.5
    against 67.6 ms at 30000 x 30000 x 1024).  Slabs of 5 tile rows (640 output rows) fill whole
    waves of thread blocks at M = 30000.
    """

    def __init__(self, M: int, N: int, K: int, device=None, slabs: int = 8):
        self.M, self.N, self.K = M, N, K
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.sizes = self.slab_plan(N, slabs)
        rows = max(self.sizes) if self.sizes else 0
        with torch.cuda.device(self.device):
            self.a_dev = torch.empty((K, M), dtype=torch.float32, device=self.device)
            self.b_dev = torch.empty((K, N), dtype=torch.float32, device=self.device)
            self.out_dev = [torch.empty((rows, M), dtype=torch.float32, device=self.device) for _ in range(2)]
            self.s_in = torch.cuda.Stream()
            self.s_out = torch.cuda.Stream()
            self.ev_in = torch.cuda.Event()
            self.ev_b = [torch.cuda.Event() for _ in self.sizes]
            self.ev_done = [torch.cuda.Event() for _ in self.sizes]
            self.ev_drained = [torch.cuda.Event() for _ in range(2)]
        self.h2d_bytes = 4 * K * (M + N)
        self.d2h_bytes = 4 * N * M

    @staticmethod
    def slab_plan(N: int, slabs: int, unit: int = 128) -> list:
        """Row counts of the launches: `slabs` equal slabs of whole 128-row units (the last one
        cut where the rows end).  Sums to N."""
        return [s for s in slab_sizes(N, max(1, slabs), unit) if s > 0]

    def run(self, a_store: torch.Tensor, b_store: torch.Tensor, out_store: torch.Tensor, p: float = 2.0,
            skip_epilogue: bool = False) -> torch.Tensor:
        """a_store (K, M), b_store (K, N), out_store (N, M): contiguous float32 host tensors.
        Returns out_store after every slab has landed (the call synchronises at the end)."""
        if tuple(a_store.shape) != (self.K, self.M) or tuple(b_store.shape) != (self.K, self.N):
            raise ValueError("a_store / b_store do not have the shapes this pipeline was built for")
        if tuple(out_store.shape) != (self.N, self.M) or not out_store.is_contiguous():
            raise ValueError("out_store must be a contiguous (N, M) tensor")
        with torch.cuda.device(self.device):
            main = torch.cuda.current_stream()
            self.s_in.wait_stream(main)
            self.s_out.wait_stream(main)
            with torch.cuda.stream(self.s_in):
                # a in one contiguous copy; then, per slab, the K x rows column block of b that the
                # slab needs (pitch N on the host, pitch N in the device copy of b)
                self.a_dev.copy_(a_store, non_blocking=True)
                self.ev_in.record(self.s_in)
                strided = b_store.is_pinned() and b_store.is_contiguous()
                if strided:
                    start = 0
                    for i, rows in enumerate(self.sizes):
                        _native.copy_2d_async(self.b_dev.data_ptr() + 4 * start, 4 * self.N,
                                              b_store.data_ptr() + 4 * start, 4 * self.N, 4 * rows, self.K,
                                              False, self.s_in.cuda_stream)
                        self.ev_b[i].record(self.s_in)
                        start += rows
                else:
                    self.b_dev.copy_(b_store, non_blocking=True)
                    for ev in self.ev_b:
                        ev.record(self.s_in)
            start = 0
            a = self.a_dev.t()
            for i, rows in enumerate(self.sizes):
                buf = self.out_dev[i % 2][:rows]
                if i == 0:
                    main.wait_event(self.ev_in)
                main.wait_event(self.ev_b[i])
                if i >= 2:
                    main.wait_event(self.ev_drained[i % 2])       # the buffer's previous slab has left
                cdist(a, self.b_dev[:, start:start + rows].t(), out=buf.t(), p=p, skip_epilogue=skip_epilogue)
                self.ev_done[i].record(main)
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(self.ev_done[i])
                    out_store[start:start + rows].copy_(buf, non_blocking=True)
                    self.ev_drained[i % 2].record(self.s_out)
                start += rows
            main.wait_stream(self.s_out)
            main.synchronize()
        return out_store
