"""CPU baseline for the benchmark: torch.cdist in float32 on the host cores, on a bounded
row slab of the benchmark workload.  TEST / BENCHMARK INFRASTRUCTURE ONLY.

The reference has no CPU implementation of its operators; what its tests and README
compare against is torch.cdist (tests/test_cdist.py:75, README.md:95-111), so that is the
CPU arm timed here, with all host threads torch will use.
"""
from __future__ import annotations

import os
import time

import torch


def time_cdist_slab(a_store: torch.Tensor, b_store: torch.Tensor, p: float, rows: int, repeats: int = 3,
                    budget_s: float = 20.0):
    """Times torch.cdist(b[:rows], a) (float32, CPU) and returns a dict with the rate in
    difference-ops per second (3 per (m, n, k) triple), the threads used and the sample.

    a_store (K, M), b_store (K, N) are the storage-layout inputs of the benchmark.
    p = 2 uses the exact-difference mode (no matrix-multiply rewrite), as the GPU kernels do.
    """
    K, M = a_store.shape
    rows = min(rows, b_store.shape[1])
    a = a_store.t().contiguous()
    b = b_store[:, :rows].t().contiguous()
    mode = "donot_use_mm_for_euclid_dist"
    torch.cdist(b[:8], a[:64], p=p, compute_mode=mode)            # warm the thread pool
    times = []
    t_begin = time.perf_counter()
    for _ in range(repeats):
        t0 = time.perf_counter()
        torch.cdist(b, a, p=p, compute_mode=mode)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_begin > budget_s:
            break
    best = min(times)
    ops = 3.0 * M * rows * K
    return {
        "value": ops / best,
        "unit": "diff-ops/s",
        "cores": torch.get_num_threads(),
        "host_cpus": os.cpu_count(),
        "kind": "port",
        "seconds": best,
        "sample": f"torch.cdist fp32 exact-difference mode on {rows} of the output rows x M={M} x K={K}, "
                  f"best of {len(times)}; full problem extrapolates linearly in rows",
    }
