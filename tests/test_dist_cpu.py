"""Row sharding over ranks, exercised with world_size-2 (and 3) Gloo process groups on CPU.
The compute step is the CPU oracle; what is under test is the partition and the gather."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kermac_b200 import dist as kdist


def test_slab_sizes_cover_and_align():
    assert kdist.slab_sizes(10, 4) == [3, 3, 3, 1]
    assert kdist.slab_sizes(30000, 8, 128) == [3840] * 7 + [3120]
    for n, w, al in [(0, 3, 128), (5, 8, 128), (1_000_000, 8, 128), (257, 2, 128), (128, 2, 128)]:
        sizes = kdist.slab_sizes(n, w, al)
        assert sum(sizes) == n and len(sizes) == w and all(s >= 0 for s in sizes)
        starts = [sum(sizes[:r]) for r in range(w)]
        assert all(st % al == 0 for st, s in zip(starts, sizes) if s > 0)
    assert kdist.shard_rows(10, 2, 4) == (6, 9)
    with pytest.raises(ValueError):
        kdist.shard_rows(10, 4, 4)
    with pytest.raises(ValueError):
        kdist.slab_sizes(10, 0)


def test_tile_ranges_are_balanced_and_cover_the_tile_order():
    assert kdist.tile_ranges(10, 4) == [(0, 3), (3, 3), (6, 2), (8, 2)]
    assert kdist.tile_ranges(2, 4) == [(0, 1), (1, 1), (2, 0), (2, 0)]
    for total, world in [(55225, 8), (55225, 4), (7, 2), (0, 3), (1, 8)]:
        ranges = kdist.tile_ranges(total, world)
        counts = [c for _, c in ranges]
        assert sum(counts) == total and max(counts) - min(counts) <= 1
        assert all(ranges[r + 1][0] == ranges[r][0] + ranges[r][1] for r in range(world - 1)) and ranges[0][0] == 0
    with pytest.raises(ValueError):
        kdist.tile_ranges(4, 0)
    # the linear tile order visits every tile once: panels of 16 tile columns, row by row inside a panel
    for tiles_m, tiles_n in [(235, 235), (3, 40), (17, 20), (1, 1), (5, 16)]:
        seen = {kdist.tile_coords(t, tiles_m, tiles_n) for t in range(tiles_m * tiles_n)}
        assert seen == {(i, j) for i in range(tiles_m) for j in range(tiles_n)}
    assert kdist.tile_coords(0, 235, 235) == (0, 0) and kdist.tile_coords(15, 235, 235) == (0, 15)
    assert kdist.tile_coords(16, 235, 235) == (1, 0) and kdist.tile_coords(16 * 235, 235, 235) == (0, 16)


def test_sharded_helpers_without_a_process_group_run_the_whole_problem():
    from oracle import kermac_oracle as ko
    g = torch.Generator().manual_seed(5)
    a, b, c, d = torch.rand(7, 20, generator=g), torch.randn(33, 7, generator=g), torch.randn(2, 7, generator=g), \
        torch.randn(33, 20, generator=g)

    def grad_compute(a_, b_, c_, d_, out):
        out.copy_(ko.cdist_grad_ref(a_, b_, c_, d_, p=1.0)[0].float())

    full = kdist.cdist_grad_sharded(a, b, c, d, p=1.0, compute=grad_compute)
    assert torch.equal(full, ko.cdist_grad_ref(a, b, c, d, p=1.0)[0].float())
    with pytest.raises(ValueError):
        kdist.cdist_grad_sharded(a, b, c, d[:30], p=1.0, compute=grad_compute)
    with pytest.raises(ValueError):
        kdist.cdist_grad_sharded(a.unsqueeze(0), b, c, d, compute=grad_compute)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_total, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import kermac_oracle as ko
        g = torch.Generator().manual_seed(0)
        a = torch.randn(70, 9, generator=g)
        b = torch.randn(n_total, 9, generator=g)
        c = torch.randn(4, 70, generator=g)

        def cdist_compute(a_, b_, out):
            out.copy_(ko.cdist_ref(a_, b_, p=2.0)[0].float())

        full = kdist.cdist_sharded(a, b, p=2.0, compute=cdist_compute)
        slab = kdist.cdist_sharded(a, b, p=2.0, compute=cdist_compute, gather=False)
        ref = ko.cdist_ref(a, b, p=2.0)[0].float().t().contiguous()       # [n][m]
        start, stop = kdist.shard_rows(n_total, rank, world, kdist.ROW_ALIGN)
        ok = torch.equal(full, ref) and torch.equal(slab, ref[start:stop])

        # chunked slab variant; on CPU ranks it takes the collective transport
        for chunks in (1, 3):
            ov = kdist.OverlappedCdist(70, n_total, "cpu", chunks=chunks)
            ok = ok and ov.transport == "collective"
            ok = ok and torch.equal(ov.run(a, b, p=2.0, compute=cdist_compute), ref)
            covered = sum(r1 - r0 for r0, r1 in ov.chunk_bounds())
            ok = ok and covered == stop - start

        def mv_compute(a_, b_, c_, out):
            out.copy_(ko.kernel_matvec_ref(a_, b_, c_, inner_operator="DIFF", inner_power="SQUARE",
                                           outer_power="SQRT", kernel_type="LAPLACE", bandwidth=8.0)[0].float())

        y = kdist.kernel_matvec_sharded(None, a, b, c, compute=mv_compute)
        yref = ko.kernel_matvec_ref(a, b, c, inner_operator="DIFF", inner_power="SQUARE", outer_power="SQRT",
                                    kernel_type="LAPLACE", bandwidth=8.0)[0].float()
        ok = ok and torch.equal(y, yref)

        # gradient sharded over the rows of b and d: a (K, M), b (N, K), c (O, K), d (N, M)
        ga = torch.rand(9, 33, generator=g)
        gc = torch.randn(3, 9, generator=g)
        gd = torch.randn(n_total, 33, generator=g)

        def grad_compute(a_, b_, c_, d_, out):
            out.copy_(ko.cdist_grad_ref(a_, b_, c_, d_, p=1.5)[0].float())

        gref = ko.cdist_grad_ref(ga, b, gc, gd, p=1.5)[0].float()
        gfull = kdist.cdist_grad_sharded(ga, b, gc, gd, p=1.5, compute=grad_compute)
        gslab = kdist.cdist_grad_sharded(ga, b, gc, gd, p=1.5, compute=grad_compute, gather=False)
        g0, g1 = kdist.shard_rows(n_total, rank, world, kdist.GRAD_ROW_ALIGN)
        ok = ok and torch.equal(gfull, gref) and torch.equal(gslab, gref[:, g0:g1])
        # the tile partition of the multicast transport: every rank marks the elements of its run of
        # tiles; summed over ranks every element of the (N, M) result is covered exactly once
        m_total = 300
        tiles_m, tiles_n = -(-m_total // kdist.TILE), -(-n_total // kdist.TILE)
        first, count = kdist.tile_ranges(tiles_m * tiles_n, world)[rank]
        cover = torch.zeros(n_total, m_total)
        for t in range(first, first + count):
            tm, tn = kdist.tile_coords(t, tiles_m, tiles_n)
            cover[tn * kdist.TILE:(tn + 1) * kdist.TILE, tm * kdist.TILE:(tm + 1) * kdist.TILE] += 1.0
        dist.all_reduce(cover)
        ok = ok and bool((cover == 1.0).all())
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world, n_total", [(2, 256), (2, 300), (3, 130), (2, 100), (2, 1000)])
def test_sharded_ops_on_gloo_ranks(world, n_total):
    # 256 rows -> equal slabs (single all_gather_into_tensor); 300 / 130 -> unequal slabs (padded
    # gather); 100 rows on 2 ranks -> the second rank owns nothing
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_total, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(results.get(r) for r in range(world)), dict(results)
