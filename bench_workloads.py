"""The non-headline workloads of `bench.py --workload {cdist_batched,grad,matvec}`.

Each function runs one workload of the hot-path scope on this rank's GPU and returns the
JSON-line dict (rank 0 prints it).  Inputs are seeded synthetic tensors with the shapes and
distributions of the benchmark configurations; timing is CUDA events on torch's current
stream, max over ranks.
"""
from __future__ import annotations

import os
import time

import torch

NOMINAL_LANE_OPS = 148 * 128 * 1.965e9          # fp32 lane-operations per second at max boost
NOMINAL_MUFU_OPS = 148 * 16 * 1.965e9


def _timed(fn, steps, warmup, barrier):
    for _ in range(warmup):
        fn()
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1) / steps


def _pipes(native):
    lane = max(native.measure_pipe(1, 8192)[0], native.measure_pipe(0, 8192)[0])
    mufu = native.measure_pipe(2, 2048)[0]
    return lane, mufu


def _e2e(host_inputs, run_on_device, out_host, steps, barrier, max_over_ranks):
    """Same op with pinned host inputs copied in and the result copied out, every step."""
    def step():
        dev = [t.cuda(non_blocking=True) for t in host_inputs]
        out = run_on_device(*dev)
        out_host.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
    for _ in range(2):
        step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / steps
    barrier()
    return ms, sum(t.numel() * 4 for t in host_inputs), out_host.numel() * 4


def cdist_batched(args, ctx):
    """a[B=4, K=512, M=16384] batched, b[1, K=512, N=16384] broadcast, U(-1,1) seed 2, p = 1.3,
    with the epilogue and with skip_epilogue."""
    import kermac_b200 as kermac
    from kermac_b200 import _native
    B, K, M, N, p = 4, 512, 16384, 16384, 1.3
    g = torch.Generator().manual_seed(2)
    a_store = 2.0 * torch.rand(B, K, M, generator=g) - 1.0
    b_store = 2.0 * torch.rand(1, K, N, generator=g) - 1.0
    a = a_store.cuda().permute(0, 2, 1)
    b = b_store.cuda().permute(0, 2, 1)
    out = torch.empty(B, N, M, device="cuda").permute(0, 2, 1)
    res = {}
    with ctx.clocks() as clocks:
        for name, skip in (("epilogue", False), ("skip_epilogue", True)):
            res[name] = _timed(lambda: kermac.cdist(a, b, out=out, p=p, skip_epilogue=skip), args.steps,
                               args.warmup, ctx.barrier)
    ms = res["epilogue"]
    ops = 3.0 * B * M * N * K
    lane, mufu = _pipes(_native)
    mufu_rate = (2.0 / 3.0) * ops / (ms * 1e-3)
    line = {
        "metric": "cdist difference-ops/s (3*L*M*N*K per step), fp32, p=1.3, batched with broadcast b",
        "value": ops / (ms * 1e-3), "unit": "diff-ops/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "cdist p=1.3 fp32 a[B=4,K=512,M=16384] b[1,K=512,N=16384] U(-1,1) seed 2",
                   "l2": "inputs 168 MB and output 4.3 GB exceed the 126 MB L2"},
        "clocks": clocks.summary(), "gpu_launches": args.steps,
        "skip_epilogue": {"ms_per_step": res["skip_epilogue"], "value": ops / (res["skip_epilogue"] * 1e-3)},
        "roofline": {"bound": "mufu", "achieved": mufu_rate / 1e12, "peak": mufu / 1e12, "unit": "T MUFU-op/s",
                     "frac": mufu_rate / mufu, "frac_of_nominal": mufu_rate / NOMINAL_MUFU_OPS,
                     "peak_source": "measured on this device (lg2.approx + ex2.approx chains)",
                     "note": "2 MUFU operations per (l, m, n, k); a fraction above 1 means part of the "
                             "exponentials ran on the FP32 pipe", "traffic": None},
    }
    if not args.no_cpu:
        rows = 64
        t0 = time.perf_counter()
        torch.cdist(b_store[0].t()[:rows].contiguous(), a_store[0].t().contiguous(), p=p)
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": 3.0 * rows * M * K / dt, "unit": "diff-ops/s", "cores": torch.get_num_threads(),
                                "kind": "port", "sample": f"torch.cdist fp32 p=1.3 on {rows} output rows of one batch entry"}
    return line


def grad(args, ctx):
    """Gradient configuration in the operator's own naming: K=30000 contracted, M=4096, N=256, O=4
    (seed 3): a (K, M) ~ U(0,1) weights, b (N, K), c (O, K), d (N, M) ~ N(0,1); p = 1.0 and p = 1.5."""
    import kermac_b200 as kermac
    from kermac_b200 import _native
    K, M, N, O = 30000, 4096, 256, 4
    g = torch.Generator().manual_seed(3)
    b = torch.randn(N, K, generator=g)
    d = torch.randn(N, M, generator=g)
    c = torch.randn(O, K, generator=g)
    a = torch.rand(M, K, generator=g).t().contiguous()
    ad, bd, cd, dd = a.cuda(), b.cuda(), c.cuda(), d.cuda()
    out = torch.empty(1, O, N, M, device="cuda")
    flush = torch.empty(64 * 1024 * 1024, device="cuda")           # 256 MB > L2

    def run(p):
        def step():
            flush.zero_()
            kermac.cdist_grad(ad, bd, cd, dd, out=out, p=p)
        return step

    def flush_only():
        flush.zero_()

    with ctx.clocks() as clocks:
        t_flush = _timed(flush_only, args.steps, args.warmup, ctx.barrier)
        ms1 = _timed(run(1.0), args.steps, args.warmup, ctx.barrier) - t_flush
        ms15 = _timed(run(1.5), args.steps, args.warmup, ctx.barrier) - t_flush
    triples = float(M) * N * K
    ops = (3.0 + 2.0 * O) * triples
    lane, mufu = _pipes(_native)
    lane_rate = (1.0 + O) * triples / (ms1 * 1e-3)            # sub + O fma lane-ops per triple (sign is a bit op)
    line = {
        "metric": "cdist_grad ops/s ((3+2*O)*M*N*K per step), fp32, p=1",
        "value": ops / (ms1 * 1e-3), "unit": "ops/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms1, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "cdist_grad fp32 a(K=30000,M=4096) U(0,1), b(N=256,K) c(O=4,K) d(N,M) N(0,1) seed 3",
                   "l2": "a 256 MB write between steps flushes the L2; its time is subtracted"},
        "clocks": clocks.summary(), "gpu_launches": 2 * args.steps,
        "p=1.5": {"ms_per_step": ms15, "value": ops / (ms15 * 1e-3),
                  "mufu_frac_of_measured": 2.0 * triples / (ms15 * 1e-3) / mufu},
        "roofline": {"bound": "fp32_simt", "achieved": lane_rate / 1e12, "peak": lane / 1e12,
                     "unit": "T fp32 lane-op/s", "frac": lane_rate / lane, "frac_of_nominal": lane_rate / NOMINAL_LANE_OPS,
                     "peak_source": "measured on this device (fma.rn.f32x2 chains)",
                     "note": "1 + O lane-operations per (m, n, k) for p = 1", "traffic": None},
    }
    if not args.no_e2e:
        out_pin = torch.empty(1, O, N, M).pin_memory()
        e_ms, h2d, d2h = _e2e([t.pin_memory() for t in (a, b, c, d)],
                              lambda a_, b_, c_, d_: kermac.cdist_grad(a_, b_, c_, d_, p=1.0), out_pin,
                              max(2, min(args.steps, 5)), ctx.barrier, ctx.max_over_ranks)
        line["e2e"] = {"value": ops / (e_ms * 1e-3), "unit": "ops/s", "ms_per_step": e_ms,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
    if not args.no_cpu:
        rows = 4
        a64 = a.double()
        t0 = time.perf_counter()
        diff = d[:rows].unsqueeze(1) - b[:rows].unsqueeze(2)                    # (rows, K, M)
        w = torch.sign(diff) * a.unsqueeze(0)
        torch.einsum('ok,nkm->onm', c, w)
        dt = time.perf_counter() - t0
        del a64
        line["cpu_baseline"] = {"value": (3.0 + 2.0 * O) * rows * M * K / dt, "unit": "ops/s",
                                "cores": torch.get_num_threads(), "kind": "port",
                                "sample": f"torch fp32 sign/einsum composition on {rows} of the {N} rows n"}
    return line


def matvec(args, ctx):
    """Fused Laplace-kernel matvec: a[K=64, M], b[K=64, N], c[O=16, M] ~ N(0,1) seed 4, sigma = 8,
    y[n, o] = sum_m exp(-|b_n - a_m|_2 / sigma) c[o, m]; rows n sharded over ranks, all-gather of y."""
    import kermac_b200 as kermac
    from kermac_b200 import _native, dist as kdist
    K, O, sigma = 64, 16, 8.0
    M, N = args.mv_m, args.mv_n
    g = torch.Generator().manual_seed(4)
    a_store = torch.randn(K, M, generator=g)
    b_store = torch.randn(K, N, generator=g)
    c = torch.randn(O, M, generator=g)
    ad, bd, cd = a_store.cuda().t(), b_store.cuda().t(), c.cuda()
    start, stop = kdist.shard_rows(N, ctx.rank, ctx.world, kdist.ROW_ALIGN)
    gather_buf, slab = kdist.gather_buffer(N, (O,), ctx.world, ctx.rank, kdist.ROW_ALIGN, torch.device("cuda"))
    launches = {"n": 0}

    def compute():
        if stop > start:
            kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, ad, bd[start:stop], cd, out=slab, bandwidth=sigma)
            launches["n"] += 1

    def job():
        compute()
        if ctx.world > 1:
            kdist.gather_rows_inplace(gather_buf, N)

    with ctx.clocks() as clocks:
        ms = ctx.max_over_ranks(_timed(job, args.steps, args.warmup, ctx.barrier))
    k_ms = ctx.max_over_ranks(_timed(compute, args.steps, 1, ctx.barrier))
    pairs = float(M) * N
    ops = (3.0 * K + 2.0 * O) * pairs
    line = {
        "metric": "kernel_matvec ops/s ((3*K+2*O)*M*N per step), fp32, Laplace L2",
        "value": ops / (ms * 1e-3), "unit": "ops/s", "n_gpus": ctx.world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": f"kernel_matvec Laplace-L2 fp32 a[K=64,M={M}] b[K=64,N={N}] c[O=16,M] N(0,1) seed 4, sigma=8",
                   "sharding": "single GPU" if ctx.world == 1 else f"rows n over {ctx.world} ranks + all-gather of y",
                   "l2": f"inputs {4 * K * (M + N) / 1e6:.0f} MB; every a tile is re-read by every row tile"},
        "clocks": clocks.summary(), "gpu_launches": args.steps,
        "compute_only": {"ms_per_step": k_ms, "value": ops / (k_ms * 1e-3)},
    }
    if ctx.rank == 0:
        lane, mufu = _pipes(_native)
        slab_pairs = float(M) * (stop - start)
        on_tensor = os.environ.get("KERMAC_B200_CONTRACTION", "auto").lower() != "fp32"
        # sub + fma per (m, n, k) on the FP32 pipe; the O products per (m, n) run there only with the
        # FP32 contraction, otherwise on the tensor cores as 3 tf32 products each
        lane_rate = (2.0 * K + (0 if on_tensor else O)) * slab_pairs / (k_ms * 1e-3)
        line["roofline"] = {"bound": "fp32_simt", "achieved": lane_rate / 1e12, "peak": lane / 1e12,
                            "unit": "T fp32 lane-op/s", "frac": lane_rate / lane,
                            "frac_of_nominal": lane_rate / NOMINAL_LANE_OPS,
                            "peak_source": "measured on this device (fma.rn.f32x2 chains)",
                            "note": ("2*K lane-operations per (m, n) pair (distance part); the O coefficient products "
                                     "per pair run on the tcgen05 tensor cores; 2 MUFU per pair run beside them") if on_tensor
                            else "2*K + O lane-operations per (m, n) pair; 2 MUFU per pair run beside them",
                            "traffic": None}
        if on_tensor:
            line["roofline"]["tensor_contraction"] = {
                "tf32_tflops_issued": 3 * 2.0 * 16 * slab_pairs / (k_ms * 1e-3) / 1e12,
                "note": "three tf32 MMAs (128 x 16 x 8) per 8 m-columns of every 128-row tile; N = 16 of the MMA is padding above O"}
        if not args.no_cpu:
            rows = 8
            a32, b32 = a_store.t().contiguous(), b_store.t()[:rows].contiguous()
            msub = min(M, 200_000)
            t0 = time.perf_counter()
            kmat = torch.exp(-torch.cdist(b32, a32[:msub], compute_mode="donot_use_mm_for_euclid_dist") / sigma)
            kmat @ c[:, :msub].t()
            dt = time.perf_counter() - t0
            line["cpu_baseline"] = {"value": (3.0 * K + 2.0 * O) * rows * msub / dt, "unit": "ops/s",
                                    "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": f"torch fp32 cdist+exp+matmul on {rows} rows n x {msub} columns m"}
    if not args.no_e2e:
        y_pin = torch.empty(stop - start, O).pin_memory()
        b_rows = b_store[:, start:stop].contiguous()
        e_ms, h2d, d2h = _e2e([a_store.pin_memory(), b_rows.pin_memory(), c.pin_memory()],
                              lambda a_, b_, c_: kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a_.t(), b_.t(),
                                                                      c_, bandwidth=sigma)[0],
                              y_pin, 2, ctx.barrier, ctx.max_over_ranks)
        line["e2e"] = {"value": ops / (e_ms * 1e-3), "unit": "ops/s", "ms_per_step": e_ms,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "note": "bytes are per rank"}
    return line
