"""The benchmark configurations beside the headline: `bench.py` runs them after its timed
region and reports them under "also"; `bench.py --workload {cdist_small,cdist_batched,grad,matvec}`
runs one of them alone.

Each function runs one configuration on this rank's GPU and returns a JSON-line dict (rank 0
prints it).  Inputs are seeded synthetic tensors with the shapes and distributions of the
benchmark configurations; timing is CUDA events on torch's current stream, max over ranks.
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


def _pipes(ctx, native):
    """Pipe rates measured once per process (bench.py's Pipes when it made one)."""
    if getattr(ctx, "pipes", None) is None:
        class P:
            pass
        p = P()
        p.lane_packed = native.measure_pipe(1, 8192)[0]
        p.lane_scalar = native.measure_pipe(0, 8192)[0]
        p.lane = max(p.lane_packed, p.lane_scalar)
        p.mufu = native.measure_pipe(2, 2048)[0]
        ctx.pipes = p
    return ctx.pipes


def _side(args):
    """True when the configuration runs as a side measurement of the headline (no e2e / CPU legs)."""
    return bool(getattr(args, "no_e2e_side", False))


def brief(line):
    """The part of a workload's line that goes under the headline's "also"."""
    drop = ("n_gpus", "steps", "warmup", "higher_is_better", "scaling", "vs_baseline", "dtype", "data", "clocks",
            "gpu_launches")
    return {k: v for k, v in line.items() if k not in drop}


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


# ------------------------------------------------------------------ fractional p: a two-pipe bound
# Per (m, n, k) element the |b - a|^p step has two routes (kermac_b200/csrc/km_common.cuh, inner_block):
#   all-MUFU    sub, lg2 (MUFU), mul by p, ex2 (MUFU), add         3 FP32-pipe lane-ops, 2 MUFU, 5 issue slots
#   polynomial  sub, lg2 (MUFU), mul by p, 2 clamps (ALU), add/sub/sub to split off the integer part,
#               5 fma of the polynomial, 1 shift (ALU), 1 fma into the sum
#                                                                   11 FP32-pipe lane-ops, 1 MUFU, 15 issue slots
# With a share x of the elements on the polynomial route the kernel cannot be faster than
#   t(x) = max( (2 - x) / MUFU rate,  (5 + 10 x) / issue rate )      per element
# (the FP32 pipe itself, (3 + 8 x) / lane rate, is always below the issue term).  The bound is the
# minimum of t over x; operand loads and the epilogue come on top and are not counted.
POW_ISSUE_SLOTS = (5.0, 15.0)        # all-MUFU, polynomial
POW_MUFU_OPS = (2.0, 1.0)
POW_POLY_SHARE = 6.0 / 8.0           # KM_POW_POLY_EIGHTHS / 8 of the build kernels as compiled


def pow_two_pipe_seconds(x, issue_rate, mufu_rate):
    """Model time per element for a polynomial share x (rates in lane-slots and MUFU ops per second)."""
    mufu = (POW_MUFU_OPS[0] * (1.0 - x) + POW_MUFU_OPS[1] * x) / mufu_rate
    issue = (POW_ISSUE_SLOTS[0] * (1.0 - x) + POW_ISSUE_SLOTS[1] * x) / issue_rate
    return max(mufu, issue), mufu, issue


def fractional_roofline(elements, seconds, pipes, share=POW_POLY_SHARE):
    """Roofline dict for `elements` (m, n, k) element-steps of |b - a|^p done in `seconds`."""
    issue_rate = pipes.lane_scalar        # one warp instruction per clock and scheduler = 32 lane-slots
    best_x, best_t = 0.0, float("inf")
    for i in range(0, 1001):
        x = i / 1000.0
        t = pow_two_pipe_seconds(x, issue_rate, pipes.mufu)[0]
        if t < best_t:
            best_x, best_t = x, t
    t_used, t_mufu, t_issue = pow_two_pipe_seconds(share, issue_rate, pipes.mufu)
    per_element = seconds / elements
    return {
        "bound": "mufu+issue (two pipes)",
        "achieved": 1.0 / per_element / 1e12, "peak": 1.0 / best_t / 1e12, "unit": "T element-steps/s",
        "frac": best_t / per_element,
        "peak_source": "min over the polynomial share x of max((2-x)/MUFU rate, (5+10x)/issue rate), both rates "
                       "measured on this device by kermac_b200_measure_pipe",
        "model_best_share": best_x, "share_in_use": share,
        "frac_of_model_at_share_in_use": t_used / per_element,
        "limiting_pipe_at_share_in_use": "issue" if t_issue >= t_mufu else "mufu",
        "all_mufu_bound_ratio": (2.0 / pipes.mufu) / per_element,
        "mufu_utilisation": (POW_MUFU_OPS[0] * (1 - share) + POW_MUFU_OPS[1] * share) / pipes.mufu / per_element,
        "issue_utilisation_model": (POW_ISSUE_SLOTS[0] * (1 - share) + POW_ISSUE_SLOTS[1] * share) / issue_rate / per_element,
        "traffic": None,
    }


def _fp32_roofline(lane_ops, seconds, pipes, note):
    rate = lane_ops / seconds
    return {"bound": "fp32_simt", "achieved": rate / 1e12, "peak": pipes.lane / 1e12, "unit": "T fp32 lane-op/s",
            "frac": rate / pipes.lane, "frac_of_nominal": rate / NOMINAL_LANE_OPS,
            "peak_source": "measured on this device (fma.rn.f32x2 chains)", "note": note, "traffic": None}


# ------------------------------------------------------------------ configuration 1
def cdist_small(args, ctx):
    """a[K=64, M=2048], b[K=64, N=2048] ~ U(0,1) seed 0, p = 2, full epilogue: the case small enough
    for a CPU; on the GPU it is launch latency and one partial wave (256 tiles on 296 block slots)."""
    import kermac_b200 as kermac
    from kermac_b200 import _native
    K, M, N = 64, 2048, 2048
    g = torch.Generator().manual_seed(0)
    a_store, b_store = torch.rand(K, M, generator=g), torch.rand(K, N, generator=g)
    a, b = a_store.cuda().t(), b_store.cuda().t()
    out = torch.empty(N, M, device="cuda").t()
    calls = 50

    def burst(p):
        def run():
            for _ in range(calls):
                kermac.cdist(a, b, out=out, p=p)
        return run

    res = {}
    with ctx.clocks() as clocks:
        for p in (2.0, 1.0, 1.3):
            res[p] = _timed(burst(p), max(3, args.steps), args.warmup, ctx.barrier) / calls
    ms = res[2.0]
    ops = 3.0 * M * N * K
    pipes = _pipes(ctx, _native)
    line = {
        "metric": "cdist difference-ops/s (3*M*N*K per call), fp32, p=2, 2048x2048x64",
        "value": ops / (ms * 1e-3), "unit": "diff-ops/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "us_per_call": {"p=2": ms * 1e3, "p=1": res[1.0] * 1e3, "p=1.3": res[1.3] * 1e3},
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "cdist p=2 fp32 a[K=64,M=2048] b[K=64,N=2048] U(0,1) seed 0, full epilogue",
                   "timing": f"{calls} back-to-back calls per timed step (launch to completion, inputs L2-resident: "
                             "the whole problem is 17 MB)"},
        "clocks": clocks.summary(), "gpu_launches": calls * args.steps,
        "roofline": {"bound": "fp32_simt", "achieved": ops / (ms * 1e-3) / 1e12, "peak": 2.0 * pipes.lane / 1e12,
                     "unit": "TFLOP/s (difference-ops)", "frac": ops / (ms * 1e-3) / (2.0 * pipes.lane),
                     "note": "latency- and wave-bound: 256 tiles of 64 k-steps; the math alone is 14 us at the pipe peak",
                     "traffic": None},
    }
    if not _side(args) and not args.no_cpu:
        t0 = time.perf_counter()
        torch.cdist(b_store.t().contiguous(), a_store.t().contiguous(), p=2.0, compute_mode="donot_use_mm_for_euclid_dist")
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": ops / dt, "unit": "diff-ops/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": "torch.cdist fp32 exact-difference mode, the whole 2048 x 2048 x 64 problem"}
    return line


# ------------------------------------------------------------------ configuration 3
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
    steps = max(2, args.steps // 3) if _side(args) else args.steps
    res = {}
    with ctx.clocks() as clocks:
        for name, skip in (("epilogue", False), ("skip_epilogue", True)):
            res[name] = _timed(lambda: kermac.cdist(a, b, out=out, p=p, skip_epilogue=skip), steps,
                               min(args.warmup, 2) if _side(args) else args.warmup, ctx.barrier)
    ms = res["epilogue"]
    elements = float(B) * M * N * K
    ops = 3.0 * elements
    pipes = _pipes(ctx, _native)
    line = {
        "metric": "cdist difference-ops/s (3*L*M*N*K per step), fp32, p=1.3, batched with broadcast b",
        "value": ops / (ms * 1e-3), "unit": "diff-ops/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "cdist p=1.3 fp32 a[B=4,K=512,M=16384] b[1,K=512,N=16384] U(-1,1) seed 2",
                   "l2": "inputs 168 MB and output 4.3 GB exceed the 126 MB L2"},
        "clocks": clocks.summary(), "gpu_launches": 2 * steps,
        "skip_epilogue": {"ms_per_step": res["skip_epilogue"], "value": ops / (res["skip_epilogue"] * 1e-3),
                          "roofline": fractional_roofline(elements, res["skip_epilogue"] * 1e-3, pipes)},
        "roofline": fractional_roofline(elements, ms * 1e-3, pipes),
    }
    if not _side(args) and not args.no_cpu:
        rows = 64
        t0 = time.perf_counter()
        torch.cdist(b_store[0].t()[:rows].contiguous(), a_store[0].t().contiguous(), p=p)
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": 3.0 * rows * M * K / dt, "unit": "diff-ops/s", "cores": torch.get_num_threads(),
                                "kind": "port", "sample": f"torch.cdist fp32 p=1.3 on {rows} output rows of one batch entry"}
    return line


# ------------------------------------------------------------------ configuration 4
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

    def run(fn):
        def step():
            flush.zero_()
            fn()
        return step

    def flush_only():
        flush.zero_()

    def ours(p):
        return lambda: kermac.cdist_grad(ad, bd, cd, dd, out=out, p=p)

    with ctx.clocks() as clocks:
        t_flush = _timed(flush_only, args.steps, args.warmup, ctx.barrier)
        ms1 = _timed(run(ours(1.0)), args.steps, args.warmup, ctx.barrier) - t_flush
        ms15 = _timed(run(ours(1.5)), args.steps, args.warmup, ctx.barrier) - t_flush
        ms17 = _timed(run(ours(1.7)), max(2, args.steps // 2), min(args.warmup, 2), ctx.barrier) - t_flush
    triples = float(M) * N * K
    ops = (3.0 + 2.0 * O) * triples
    pipes = _pipes(ctx, _native)
    line = {
        "metric": "cdist_grad ops/s ((3+2*O)*M*N*K per step), fp32, p=1",
        "value": ops / (ms1 * 1e-3), "unit": "ops/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms1, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "cdist_grad fp32 a(K=30000,M=4096) U(0,1), b(N=256,K) c(O=4,K) d(N,M) N(0,1) seed 3",
                   "l2": "a 256 MB write between steps flushes the L2; its time is subtracted"},
        "clocks": clocks.summary(), "gpu_launches": 2 * args.steps,
        "p=1.5": {"ms_per_step": ms15, "value": ops / (ms15 * 1e-3),
                  "roofline": {"bound": "mufu", "achieved": triples / (ms15 * 1e-3) / 1e12, "peak": pipes.mufu / 1e12,
                               "unit": "T MUFU-op/s", "frac": triples / (ms15 * 1e-3) / pipes.mufu,
                               "fp32_lane_utilisation": (2.0 + O) * triples / (ms15 * 1e-3) / pipes.lane,
                               "note": "p - 1 = 1/2: |x|^(p-1) is one sqrt.approx, 1 MUFU operation per (m, n, k); "
                                       "2 + O FP32 lane-operations beside it", "traffic": None}},
        "p=1.7": {"ms_per_step": ms17, "value": ops / (ms17 * 1e-3),
                  "roofline": {"bound": "mufu", "achieved": 1.75 * triples / (ms17 * 1e-3) / 1e12, "peak": pipes.mufu / 1e12,
                               "unit": "T MUFU-op/s", "frac": 1.75 * triples / (ms17 * 1e-3) / pipes.mufu,
                               "note": "general p: lg2 and ex2 per (m, n, k); one pair in four takes its ex2 on the FP32 "
                                       "pipe, so 1.75 MUFU operations per (m, n, k)", "traffic": None}},
        # sub + O fma lane-operations per (m, n, k); the sign flip is a bit operation on the ALU pipe
        "roofline": _fp32_roofline((1.0 + O) * triples, ms1 * 1e-3, pipes, "1 + O lane-operations per (m, n, k) for p = 1"),
    }
    # what the k step's instruction mix sustains from registers alone (no loads, staging or barriers):
    # its packed FMAs read three different register pairs and do not issue at the packed rate
    step_packed = _native.measure_pipe(6, 2048)[0]
    step_scalar = _native.measure_pipe(7, 2048)[0]
    line["roofline"]["inner_step_ceiling_lane_ops"] = step_packed
    line["roofline"]["frac_of_inner_step_ceiling"] = (1.0 + O) * triples / (ms1 * 1e-3) / step_packed
    line["roofline"]["inner_step_ceiling_scalar_fma_lane_ops"] = step_scalar
    # 32 and 64 channels: the tensor-core kernel (the automatic choice from 17 channels on) next to the FP32 kernel.
    # Its bound is the tensor pipe at the rate narrow MMAs get: a 128 x 8 tf32 MMA of up to 64 output
    # columns holds the pipe ~45 cycles; two of them (head and remainder of the weights) per 128 pairs x 8 k.
    few = max(2, args.steps // 3)
    mma_rates = [_native.measure_pipe(kind, 4096)[0] for kind in (8, 9, 10, 11)]   # 128 x {32, 64, 128, 256} x 8
    for O2 in (32, 64):
        c2 = torch.randn(O2, K, generator=g).cuda()
        out2 = torch.empty(1, O2, N, M, device="cuda")
        t_fp = _timed(run(lambda: kermac.cdist_grad(ad, bd, c2, dd, out=out2, p=1.0, contraction="fp32")), few, 1,
                      ctx.barrier) - t_flush
        fp_out = out2.clone()
        t_tc = _timed(run(lambda: kermac.cdist_grad(ad, bd, c2, dd, out=out2, p=1.0, contraction="tensor")), few, 1,
                      ctx.barrier) - t_flush
        # per 128 pairs x 8 k: one MMA of 2 O2 columns (heads) and one of O2 columns (remainders)
        per_step = float(M) * N / 128.0 * (K / 8.0)
        wide, narrow = (mma_rates[1], mma_rates[0]) if O2 == 32 else (mma_rates[2], mma_rates[1])
        t_bound = per_step / wide + per_step / narrow
        line[f"O={O2}"] = {"fp32_kernel_ms": t_fp, "tensor_kernel_ms": t_tc, "ratio": t_fp / t_tc,
                           "max_abs_diff_over_max": float((out2 - fp_out).abs().max() / fp_out.abs().max()),
                           "device_error_flag": _native.device_error_flag(),
                           "roofline": {"bound": "tensor", "achieved": 2.0 * per_step / (t_tc * 1e-3) / 1e9,
                                        "peak": 2.0 * per_step / t_bound / 1e9, "unit": "G narrow-MMA/s",
                                        "frac": t_bound / (t_tc * 1e-3), "traffic": None,
                                        "peak_source": "measured on this device by kermac_b200_measure_pipe kinds 8-11",
                                        "mma_per_s_n32_n64_n128_n256": mma_rates,
                                        "note": "tcgen05.mma kind::tf32 128 x N x 8 holds the tensor pipe ~45 cycles up to "
                                                "N = 64 and N / 2 cycles from 128 on; per 128 pairs x 8 k one of 2 O columns "
                                                "(heads of the weights) and one of O columns (remainders)"}}
        del c2, out2, fp_out
    if not args.no_ref_gpu:
        from baseline import ref_kernels
        if ref_kernels.available():
            o_ref = torch.empty(O, N, M, device="cuda")
            ref = {}
            for p, ours_ms in ((1.0, ms1), (1.5, ms15)):
                t = _timed(run(lambda: ref_kernels.ref_cdist_grad(ad, bd, cd, dd, o_ref, p)), max(2, args.steps // 3), 1,
                           ctx.barrier) - t_flush
                kermac.cdist_grad(ad, bd, cd, dd, out=out, p=p)
                scale = float(o_ref.abs().max())
                ref[f"p={p:g}"] = {"reference_kernel_ms": t, "ratio": t / ours_ms,
                                   "max_abs_diff_over_max": float((out[0] - o_ref).abs().max()) / scale}
            line["ref_gpu"] = ref
        else:
            line["ref_gpu"] = {"unavailable": "baseline/_ref holds no cubin of the reference's kernels"}
    if not _side(args) and not args.no_e2e:
        out_pin = torch.empty(1, O, N, M).pin_memory()
        e_ms, h2d, d2h = _e2e([t.pin_memory() for t in (a, b, c, d)],
                              lambda a_, b_, c_, d_: kermac.cdist_grad(a_, b_, c_, d_, p=1.0), out_pin,
                              max(2, min(args.steps, 5)), ctx.barrier, ctx.max_over_ranks)
        line["e2e"] = {"value": ops / (e_ms * 1e-3), "unit": "ops/s", "ms_per_step": e_ms,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
    if not _side(args) and not args.no_cpu:
        rows = 4
        t0 = time.perf_counter()
        diff = d[:rows].unsqueeze(1) - b[:rows].unsqueeze(2)                    # (rows, K, M)
        w = torch.sign(diff) * a.unsqueeze(0)
        torch.einsum('ok,nkm->onm', c, w)
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": (3.0 + 2.0 * O) * rows * M * K / dt, "unit": "ops/s",
                                "cores": torch.get_num_threads(), "kind": "port",
                                "sample": f"torch fp32 sign/einsum composition on {rows} of the {N} rows n"}
    return line


# ------------------------------------------------------------------ configuration 5
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
    steps = max(1, args.mv_steps) if _side(args) else args.steps
    warmup = 1 if _side(args) else args.warmup

    def compute():
        if stop > start:
            kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, ad, bd[start:stop], cd, out=slab, bandwidth=sigma)
            launches["n"] += 1

    def job():
        compute()
        if ctx.world > 1:
            kdist.gather_rows_inplace(gather_buf, N)

    with ctx.clocks() as clocks:
        ms = ctx.max_over_ranks(_timed(job, steps, warmup, ctx.barrier))
    k_ms = ctx.max_over_ranks(_timed(compute, steps, 0, ctx.barrier))
    pairs = float(M) * N
    ops = (3.0 * K + 2.0 * O) * pairs
    line = {
        "metric": "kernel_matvec ops/s ((3*K+2*O)*M*N per step), fp32, Laplace L2",
        "value": ops / (ms * 1e-3), "unit": "ops/s", "n_gpus": ctx.world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": f"kernel_matvec Laplace-L2 fp32 a[K=64,M={M}] b[K=64,N={N}] c[O=16,M] N(0,1) seed 4, sigma=8",
                   "sharding": "single GPU" if ctx.world == 1 else f"rows n over {ctx.world} ranks + all-gather of y",
                   "l2": f"inputs {4 * K * (M + N) / 1e6:.0f} MB; every a tile is re-read by every row tile"},
        "clocks": clocks.summary(), "gpu_launches": steps,
        "compute_only": {"ms_per_step": k_ms, "value": ops / (k_ms * 1e-3)},
    }
    pipes = _pipes(ctx, _native)
    slab_pairs = float(M) * ctx.max_over_ranks(float(stop - start))
    on_tensor = os.environ.get("KERMAC_B200_CONTRACTION", "auto").lower() != "fp32"
    # sub + fma per (m, n, k) on the FP32 pipe; the O products per (m, n) run there only with the
    # FP32 contraction, otherwise on the tensor cores as 3 tf32 products each
    line["roofline"] = _fp32_roofline(
        (2.0 * K + (0 if on_tensor else O)) * slab_pairs, k_ms * 1e-3, pipes,
        ("2*K lane-operations per (m, n) pair (distance part); the O coefficient products per pair run on the tcgen05 "
         "tensor cores; 2 MUFU per pair run beside them") if on_tensor
        else "2*K + O lane-operations per (m, n) pair; 2 MUFU per pair run beside them")
    if on_tensor:
        line["roofline"]["tensor_contraction"] = {
            "tf32_tflops_issued": 3 * 2.0 * 16 * slab_pairs / (k_ms * 1e-3) / 1e12,
            "note": "three tf32 MMAs (128 x 16 x 8) per 8 m-columns of every 128-row tile; N = 16 of the MMA is padding above O"}
    if ctx.world > 1:
        line["verified"] = verify_matvec(ctx, gather_buf[:N], ad, bd, cd, sigma)
    if ctx.rank == 0 and not _side(args) and not args.no_cpu:
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
    if not _side(args) and not args.no_e2e:
        y_pin = torch.empty(stop - start, O).pin_memory()
        b_rows = b_store[:, start:stop].contiguous()
        e_ms, h2d, d2h = _e2e([a_store.pin_memory(), b_rows.pin_memory(), c.pin_memory()],
                              lambda a_, b_, c_: kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a_.t(), b_.t(),
                                                                      c_, bandwidth=sigma)[0],
                              y_pin, 2, ctx.barrier, ctx.max_over_ranks)
        line["e2e"] = {"value": ops / (e_ms * 1e-3), "unit": "ops/s", "ms_per_step": e_ms,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "note": "bytes are per rank"}
    return line


# ------------------------------------------------------------------ the reference's own kernels, same GPU
def ref_gpu_cdist(a, b, slab, also, head_p, head_ms, ops_total):
    """Times the reference's cute_build_kernel instantiations (baseline/_ref, NVRTC-built from the
    reference's sources for sm_100 as its JIT would) on the benchmark's own device tensors, and
    compares the values with ours.  `slab` holds our result for the last p that ran; it is reused."""
    from baseline import ref_kernels
    import kermac_b200 as kermac
    if not ref_kernels.available():
        return {"unavailable": "baseline/_ref holds no cubin of the reference's kernels (built by "
                               "baseline/build_ref_cubin.py where the reference checkout is present)"}
    ours_ms = {head_p: head_ms}
    for key, entry in also.items():
        if key.startswith("p=") and "cdist" not in key:
            ours_ms[float(key[2:])] = entry["ms_per_step"]
    out_ref = torch.empty_like(slab)
    res = {"what": "cute_build_kernel (ALIGN_4 instantiation, the one try_to_align=True selects), launched with the grid "
                   "and arguments of src/kermac/build_a_kernel.py:348-390; same inputs, same GPU, CUDA events"}
    for p in (1.0, 2.0, 1.3):
        steps = 3 if p != 1.3 else 2
        t = _timed(lambda: ref_kernels.ref_cdist(a, b, out_ref.t(), p, aligned=True), steps, 1, lambda: None)
        kermac.cdist(a, b, out=slab.t(), p=p)
        rel = float(((slab - out_ref).abs() / out_ref.abs().clamp_min(1e-30)).max())
        entry = {"reference_kernel_ms": t, "value": ops_total / (t * 1e-3), "max_rel_diff_vs_ours": rel}
        if p in ours_ms:
            entry["ours_ms"] = ours_ms[p]
            entry["ratio"] = t / ours_ms[p]
        res[f"p={p:g}"] = entry
    return res


# ------------------------------------------------------------------ N > 1: is the exchanged result right?
def _sample_rows(n_total, world, per_slab, seed):
    """`per_slab` row indices out of every rank's slab of rows (same on every rank)."""
    from kermac_b200 import dist as kdist
    g = torch.Generator().manual_seed(seed)
    sizes = kdist.slab_sizes(n_total, world, kdist.ROW_ALIGN)
    rows, start = [], 0
    for size in sizes:
        if size > 0:
            pick = torch.randint(0, size, (min(per_slab, size),), generator=g) + start
            rows.append(pick)
            # the slab's first and last row sit on the seams between ranks
            rows.append(torch.tensor([start, start + size - 1]))
        start += size
    return torch.unique(torch.cat(rows)) if rows else torch.zeros(0, dtype=torch.long)


def verify_sharded(ctx, cyc, a, b):
    """Every rank compares sampled rows of the exchanged cdist result (rows from every rank's part of
    the output) with its own single-GPU cdist of those rows, then does the same for a sharded
    cdist_grad.  Bitwise for p = 1 and p = 2 (the same sequential sum over k wherever a tile runs);
    to 2e-6 relative for p = 1.3, whose exp2 route depends on the position inside a tile."""
    import kermac_b200 as kermac
    from kermac_b200 import _native, dist as kdist
    N = b.size(0)
    rows = _sample_rows(N, ctx.world, 32, seed=11).to(a.device)
    b_rows = b[rows]                                   # (R, K): k-contiguous copy of the sampled points
    report = {"rows_sampled": int(rows.numel()), "partition": cyc.partition, "transport": cyc.transport}
    ok_all = True
    for p in (1.0, 2.0, 1.3):
        full = cyc.run(a, b, p=p, gather=True)
        torch.cuda.synchronize()
        single = kermac.cdist(a, b_rows, p=p)[0].t()   # (R, M)
        got = full[rows]
        if p == 1.3:
            err = float(((got - single).abs() / single.abs().clamp_min(1e-30)).max())
            ok = err <= 2e-6
            report[f"p={p:g}"] = {"max_rel_diff": err, "ok": ok}
        else:
            ok = bool(torch.equal(got, single))
            report[f"p={p:g}"] = {"bitwise": ok, "ok": ok}
        ok_all = ok_all and ok
    # the gradient sharded over the rows of b and d
    g = torch.Generator().manual_seed(12)
    Kg, Mg, Ng, Og = 2048, 512, 256, 4
    ga = torch.rand(Kg, Mg, generator=g).to(a.device)
    gb = torch.randn(Ng, Kg, generator=g).to(a.device)
    gc = torch.randn(Og, Kg, generator=g).to(a.device)
    gd = torch.randn(Ng, Mg, generator=g).to(a.device)
    for p in (1.0, 1.5):
        full = kdist.cdist_grad_sharded(ga, gb, gc, gd, p=p)
        single = kermac.cdist_grad(ga, gb, gc, gd, p=p)[0]
        err = float((full - single).abs().max()) / float(single.abs().max())
        ok = err <= 2e-5       # the automatic k split may differ between the sharded and the whole problem
        report[f"cdist_grad p={p:g}"] = {"max_abs_diff_over_max": err, "ok": ok}
        ok_all = ok_all and ok
    flag_clear = _native.device_error_flag() == 0
    report["device_error_flag_clear_on_every_rank"] = ctx.all_ranks_ok(flag_clear)
    report["ok"] = ctx.all_ranks_ok(ok_all and flag_clear)
    return report


def verify_matvec(ctx, y_full, a, b, c, sigma):
    """Sampled rows of the gathered y against this rank's own kernel_matvec of those rows."""
    import kermac_b200 as kermac
    from kermac_b200 import _native
    rows = _sample_rows(b.size(0), ctx.world, 16, seed=13).to(a.device)
    b_rows = b[rows]
    single = kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a, b_rows, c, bandwidth=sigma)[0]
    err = float((y_full[rows] - single).abs().max()) / float(single.abs().max())
    # the automatic split over m depends on the number of row tiles: sums of 10^6 fp32 terms grouped
    # differently agree to a few 1e-6 of the largest entry (the oracle tolerance of the tests is 5e-5)
    ok = err <= 2e-5
    flag_clear = _native.device_error_flag() == 0
    return {"rows_sampled": int(rows.numel()), "max_abs_diff_over_max": err,
            "ok": ctx.all_ranks_ok(ok and flag_clear)}
