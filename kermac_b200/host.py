"""`cdist` for operands and results that live in host memory.

The kermac API takes device tensors (src/kermac/cdist.py:9-83 of the reference); a caller
whose data sits in host memory pays a host-to-device copy of a and b and a device-to-host
copy of the (much larger) distance matrix around it.  `HostCdist` keeps device buffers and
streams for one problem shape and overlaps the three phases: the output rows are cut into
slabs, and while slab i is computed, slab i-1 drains to the host.  Nothing here changes what is computed: each slab is a plain `cdist` call.
"""
from __future__ import annotations

import torch

from .cdist import cdist
from .dist import slab_sizes

__all__ = ["HostCdist"]


class HostCdist:
    """Pipelined host-to-host cdist for a[K, M], b[K, N] -> out[N, M] (storage layouts).

    Host tensors should be pinned, otherwise the copies do not overlap.  `slabs` is the
    number of row slabs of the output; two slab buffers rotate on the device.
    """

    def __init__(self, M: int, N: int, K: int, device=None, slabs: int = 8):
        self.M, self.N, self.K = M, N, K
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.sizes = [s for s in slab_sizes(N, max(1, slabs), 128) if s > 0]
        rows = max(self.sizes) if self.sizes else 0
        with torch.cuda.device(self.device):
            self.a_dev = torch.empty((K, M), dtype=torch.float32, device=self.device)
            self.b_dev = torch.empty((K, N), dtype=torch.float32, device=self.device)
            self.out_dev = [torch.empty((rows, M), dtype=torch.float32, device=self.device) for _ in range(2)]
            self.s_in = torch.cuda.Stream()
            self.s_out = torch.cuda.Stream()
            self.ev_in = torch.cuda.Event()
            self.ev_done = [torch.cuda.Event() for _ in self.sizes]
            self.ev_drained = [torch.cuda.Event() for _ in range(2)]
        self.h2d_bytes = 4 * K * (M + N)
        self.d2h_bytes = 4 * N * M

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
                # two contiguous copies (a strided host slice would be staged through a
                # temporary); at ~4 K (M + N) bytes they are small next to the output
                self.a_dev.copy_(a_store, non_blocking=True)
                self.b_dev.copy_(b_store, non_blocking=True)
                self.ev_in.record(self.s_in)
            start = 0
            a = self.a_dev.t()
            for i, rows in enumerate(self.sizes):
                buf = self.out_dev[i % 2][:rows]
                if i == 0:
                    main.wait_event(self.ev_in)
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
