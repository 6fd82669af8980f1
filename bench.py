"""Benchmark of the fused distance hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--p 1.0]

One "step" of the headline is one full cdist over a[K=1024, M=30000], b[K=1024, N=30000],
float32, entries N(0,1) from seed 1, out[N, M] (3.6 GB), epilogue on, default p = 1.0.  At
N > 1 GPUs the output is sharded over ranks (fixed total work: strong scaling) and the step
ends with the full result present on every rank.

Prints ONE JSON line (rank 0):
  value         difference-ops per second, 3*M*N*K per step, inputs resident on the device
  e2e           same metric through kermac_b200.HostCdist: pinned host inputs copied in, result
                copied out to pinned host memory, every step
  roofline      the cdist kernel against the FP32 pipe peak measured on this device
  cpu_baseline  torch.cdist float32 on the host cores over a bounded row slab
  also          every other benchmark configuration, outside the headline's timed region, each
                with ms_per_step, value and its own roofline:
                  the same inputs at p = 2 and p = 1.3, cdist(a, a);
                  the small 2048 x 2048 x 64 case (latency);
                  the batched fractional-p case with and without the epilogue;
                  cdist_grad at p = 1 and p = 1.5;
                  kernel_matvec at M = N = 10^6, rows sharded over the ranks, all-gather included;
                  ref_gpu: the reference's own CUDA kernels (compiled from its sources into
                  baseline/_ref by baseline/build_ref_cubin.py) on the same inputs and GPU
  verified      (N > 1) every rank compares sampled rows of every peer's part of the exchanged
                results with its own single-GPU computation of those rows, and reports its
                device error flag
`--impl reference` times the CPU arm alone (the reference has no CPU implementation of its own;
torch.cdist is what its tests and README compare against).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

K_DIM, M_DIM, N_DIM, SEED = 1024, 30000, 30000, 1
WORKLOAD = "cdist fp32 a[K=1024,M=30000] b[K=1024,N=30000] N(0,1) seed 1, out[N,M], full epilogue"
# dram__bytes_read.sum + dram__bytes_write.sum of the cdist kernel, per launch.  Captured with ncu on
# M = N = 8192, K = 1024 (profiles/), where it is 390 MB against 335 MB algorithmic (67 MB in + 268 MB out);
# scaled to the full launch by the output and input bytes, which is what the traffic is proportional to.
TRAFFIC_BYTES_PER_LAUNCH = int(390e6 / 335e6 * 4 * (M_DIM * N_DIM + K_DIM * (M_DIM + N_DIM)))
TRAFFIC_NOTE = ("scaled from an ncu capture at 8192x8192x1024 (390 MB measured vs 335 MB algorithmic); "
                "HBM is not the bound of this kernel")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--p", type=float, default=1.0)
    ap.add_argument("--m", type=int, default=M_DIM)
    ap.add_argument("--n", type=int, default=N_DIM)
    ap.add_argument("--k", type=int, default=K_DIM)
    ap.add_argument("--no-also", action="store_true", help="skip every side measurement")
    ap.add_argument("--no-configs", action="store_true",
                    help="keep the p=2 / p=1.3 side measurements but skip the other benchmark configurations")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-ref-gpu", action="store_true")
    ap.add_argument("--cpu-rows", type=int, default=512)
    ap.add_argument("--workload", default="cdist",
                    choices=["cdist", "cdist_small", "cdist_batched", "grad", "matvec"],
                    help="cdist is the headline workload; the others run one of the remaining configurations alone")
    ap.add_argument("--mv-m", type=int, default=1_000_000, help="matvec: number of points a")
    ap.add_argument("--mv-n", type=int, default=1_000_000, help="matvec: number of points b")
    ap.add_argument("--mv-steps", type=int, default=2, help="matvec: timed steps (one step is seconds at full size)")
    return ap.parse_args()


def make_inputs(m, n, k):
    g = torch.Generator().manual_seed(SEED)
    a_store = torch.randn(k, m, generator=g, dtype=torch.float32)
    b_store = torch.randn(k, n, generator=g, dtype=torch.float32)
    return a_store, b_store


def use_all_host_threads():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to every rank; the CPU arms are meant to
    use the cores this process may run on, at every N."""
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    torch.set_num_threads(max(1, cores))
    return torch.get_num_threads()


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.lines = []
        self.proc = None
        self.thread = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        busy = [c for c, w in zip(sm, power) if w >= 0.5 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "power_w_max": max(power),
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args):
    """torch.cdist float32 on the host cores, a bounded row slab per step (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = use_all_host_threads()
    from oracle import cpu_baseline
    a_store, b_store = make_inputs(args.m, args.n, args.k)
    rows = min(args.cpu_rows, args.n)
    for _ in range(max(args.warmup, 0)):
        cpu_baseline.time_cdist_slab(a_store, b_store, args.p, rows=min(rows, 64), repeats=1)
    times = []
    for _ in range(args.steps):
        r = cpu_baseline.time_cdist_slab(a_store, b_store, args.p, rows=rows, repeats=1)
        times.append(r["seconds"])
    per_step = sum(times) / len(times)
    value = 3.0 * args.m * rows * args.k / per_step
    line = {
        "impl": "reference", "metric": metric_name(args.p), "value": value, "unit": "diff-ops/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args, args.gpus),
        "cpu_baseline": {"value": value, "unit": "diff-ops/s", "cores": threads,
                         "kind": "port", "sample": r["sample"]},
        "e2e": {"value": value, "unit": "diff-ops/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# Best kermac.cdist time the reference publishes for this problem size (README.md:95-111 of the
# reference; none of it on B200): p -> (milliseconds, GPU).
PUBLISHED_MS = {1.0: (76.0, "RTX 4090"), 1.3: (350.0, "RTX 4090"), 2.0: (77.0, "RTX 4090")}


def vs_published(args, world, value):
    """value / published difference-ops per second, for the exact published problem on one GPU."""
    if (args.m, args.n, args.k) != (M_DIM, N_DIM, K_DIM) or args.p not in PUBLISHED_MS:
        return None
    return value / (3.0 * M_DIM * N_DIM * K_DIM / (PUBLISHED_MS[args.p][0] * 1e-3))


def metric_name(p):
    return f"cdist difference-ops/s (3*M*N*K per step), fp32, p={p:g}"


def config_dict(args, world):
    return {"workload": WORKLOAD if (args.m, args.n, args.k) == (M_DIM, N_DIM, K_DIM)
            else f"cdist fp32 a[K={args.k},M={args.m}] b[K={args.k},N={args.n}] N(0,1) seed 1",
            "p": args.p, "M": args.m, "N": args.n, "K": args.k,
            "sharding": "single GPU" if world == 1 else
            f"the 128 x 128 output tiles in equal contiguous runs over {world} ranks; the kernel writes its tiles to "
            "the NVSwitch multicast address of the result buffer (multimem.st), so every rank holds the full result "
            "when it ends",
            "l2": "inputs (246 MB) and output (3.6 GB) exceed the 126 MB L2; no flush needed between steps",
            "vs_baseline_is": "value / the best kermac.cdist throughput the reference publishes for this size and p "
                              "(README table: %s ms on %s)" % PUBLISHED_MS.get(args.p, ("n/a", "n/a"))}


def timed_steps(fn, steps, warmup, barrier):
    """Runs fn() warmup + steps times; returns (total ms of the timed steps on this rank's device)."""
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
    return e0.elapsed_time(e1)


def emit(line):
    """Writes the one JSON line to the real stdout (libraries that print to fd 1 were sent to stderr)."""
    os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())


_REAL_STDOUT = os.dup(1)


class Pipes:
    """Arithmetic-pipe rates of this device at the clocks it runs at now (register-only kernels)."""

    def __init__(self, native):
        self.lane_packed = native.measure_pipe(1, 8192)[0]
        self.lane_scalar = native.measure_pipe(0, 8192)[0]
        self.mufu = native.measure_pipe(2, 2048)[0]
        self.lane = max(self.lane_packed, self.lane_scalar)
        self.loop_p2 = native.measure_pipe(4, 2048)[0]
        self.loop_p1 = native.measure_pipe(5, 2048)[0]


def cdist_roofline(p, ops, seconds, pipes):
    """Roofline dict of one cdist launch that performed `ops` difference-ops in `seconds`."""
    import bench_workloads
    achieved = ops / seconds
    if p in (1.0, 2.0):
        loop = pipes.loop_p1 if p == 1.0 else pipes.loop_p2
        return {
            "bound": "fp32_simt", "achieved": achieved / 1e12, "peak": 2.0 * pipes.lane / 1e12,
            "unit": "TFLOP/s (difference-ops)", "frac": achieved / (2.0 * pipes.lane),
            "peak_source": "measured on this device by kermac_b200_measure_pipe (fma.rn.f32x2 chains), x2 flop per lane-op",
            "frac_of_nominal_74.45": achieved / (148 * 128 * 2 * 1.965e9),
            "fma_pipe_lane_utilisation": (2.0 / 3.0) * achieved / pipes.lane,
            "inner_loop_ceiling_lane_ops": loop,
            "frac_of_inner_loop_ceiling": (2.0 / 3.0) * achieved / loop,
            "lane_ops_scalar": pipes.lane_scalar, "lane_ops_packed": pipes.lane_packed,
        }
    return bench_workloads.fractional_roofline(ops / 3.0, seconds, pipes)


def main():
    args = parse_args()
    sys.stdout.flush()
    os.dup2(2, 1)          # NCCL and friends print banners on fd 1; the JSON line must stand alone
    if args.impl == "reference":
        reference_arm(args)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: kermac_b200 has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    import kermac_b200 as kermac
    from kermac_b200 import _native, dist as kdist
    from kermac_b200.host import HostCdist
    import bench_workloads

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_ranks_ok(flag: bool) -> bool:
        if world == 1:
            return bool(flag)
        t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    class Ctx:
        pass
    ctx = Ctx()
    ctx.rank, ctx.world, ctx.barrier, ctx.max_over_ranks, ctx.device = rank, world, barrier, max_over_ranks, device
    ctx.clocks = lambda: ClockSampler(local_rank)
    ctx.all_ranks_ok = all_ranks_ok
    ctx.pipes = None

    def finish(line):
        # a bounded wait that ran out on ANY rank leaves stale rows behind: every rank reads its own flag
        clean = all_ranks_ok(_native.device_error_flag() == 0)
        if rank == 0:
            assert clean, "a bounded wait inside a kernel ran out on some rank"
            emit(line)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()

    if args.workload != "cdist":
        line = getattr(bench_workloads, args.workload)(args, ctx)
        finish(line)
        return

    M, N, K = args.m, args.n, args.k
    a_store, b_store = make_inputs(M, N, K)
    a_dev, b_dev = a_store.to(device), b_store.to(device)
    a, b = a_dev.t(), b_dev.t()                    # API tensors (M, K), (N, K), m / n contiguous
    launches = {"n": 0}
    if world == 1:
        start, stop = 0, N
        share = 1.0
        slab = torch.empty((N, M), dtype=torch.float32, device=device)

        def compute_step(p):
            def step():
                kermac.cdist(a, b, out=slab.t(), p=p)
                launches["n"] += 1
            return step

        job_step = compute_step
    else:
        # one launch per rank over its run of output tiles; the kernel's stores go to the multicast
        # address of the symmetric result buffer, so the exchange happens while it computes
        cyc = kdist.OverlappedCdist(M, N, device, chunks=int(os.environ.get("KM_DIST_CHUNKS", "8")),
                                    transport=os.environ.get("KM_DIST_TRANSPORT", "auto"))
        share = cyc.work_share()
        start, stop = kdist.shard_rows(N, rank, world, kdist.ROW_ALIGN)
        slab = None

        def compute_step(p):
            return lambda: cyc.run(a, b, p=p, gather=False)

        def job_step(p):
            return lambda: cyc.run(a, b, p=p, gather=True)

    ops_total = 3.0 * M * N * K
    with ClockSampler(local_rank) as clocks:
        launches["n"] = 0
        if world > 1:
            cyc.launch_count = 0
        ms = max_over_ranks(timed_steps(job_step(args.p), args.steps, args.warmup, barrier))
        issued = launches["n"] if world == 1 else cyc.launch_count
        timed_launches = issued * args.steps // (args.steps + args.warmup)
    ms_per_step = ms / args.steps
    value = ops_total / (ms_per_step * 1e-3)
    clock_info = clocks.summary()

    # kernel-only time (no exchange) on this rank's share, for the roofline
    k_ms = max_over_ranks(timed_steps(compute_step(args.p), args.steps, 1, barrier)) / args.steps
    share = max_over_ranks(share)          # the slowest rank is the one with the largest share
    share_ops = ops_total * share

    line = {
        "metric": metric_name(args.p), "value": value, "unit": "diff-ops/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": vs_published(args, world, value), "dtype": "f32", "data": "synthetic",
        "config": config_dict(args, world), "clocks": clock_info, "gpu_launches": timed_launches,
        "compute_only": {"ms_per_step": k_ms, "value": ops_total / (k_ms * 1e-3),
                         "note": "cdist kernel on this rank's share of the output, max over ranks, no exchange"},
    }
    if world > 1:
        line["config"]["transport"] = cyc.transport
        line["config"]["partition"] = cyc.partition

    pipes = Pipes(_native)
    ctx.pipes = pipes
    roof = cdist_roofline(args.p, share_ops, k_ms * 1e-3, pipes)
    roof["traffic"] = TRAFFIC_BYTES_PER_LAUNCH if (M, N, K) == (M_DIM, N_DIM, K_DIM) and world == 1 else None
    roof["traffic_note"] = TRAFFIC_NOTE
    roof["hbm_gbs_algorithmic"] = 4.0 * (M * N * share + K * (M + N * share)) / (k_ms * 1e-3) / 1e9
    line["roofline"] = roof

    also = {}
    if not args.no_also:
        for p in (2.0, 1.3):
            if p == args.p:
                continue
            steps = args.steps if p == 2.0 else max(2, args.steps // 3)
            t = max_over_ranks(timed_steps(compute_step(p), steps, 1, barrier)) / steps
            also[f"p={p:g}"] = {"ms_per_step": t, "value": ops_total / (t * 1e-3), "unit": "diff-ops/s",
                                "note": "compute only (no exchange)",
                                "roofline": cdist_roofline(p, share_ops, t * 1e-3, pipes)}
        if world == 1 and M == N:
            # the same matrix on both sides: one triangle of tiles is computed and mirrored
            def self_step():
                kermac.cdist(a, a, out=slab.t(), p=args.p)
            t = timed_steps(self_step, args.steps, 1, barrier) / args.steps
            also[f"p={args.p:g} cdist(a, a)"] = {"ms_per_step": t, "value": ops_total / (t * 1e-3), "unit": "diff-ops/s",
                                                 "note": "a and b the same matrix: symmetric build, 3*M*N*K still counted"}
        if world == 1 and not args.no_ref_gpu:
            also["ref_gpu"] = bench_workloads.ref_gpu_cdist(a, b, slab, also, args.p, ms_per_step, ops_total)

    if world > 1:
        line["verified"] = bench_workloads.verify_sharded(ctx, cyc, a, b)

    if not args.no_e2e:
        # slabs of 5 tile rows: 5 x ceil(M / 128) tiles are a whole number of waves of thread blocks at M = 30000
        pipe = HostCdist(M, stop - start, K, device=device, slabs=max(1, round((stop - start) / 640)))
        a_pin = a_store.pin_memory()
        b_pin = b_store[:, start:stop].contiguous().pin_memory()
        out_pin = torch.empty((stop - start, M), dtype=torch.float32).pin_memory()
        slab = None
        if world > 1:
            cyc.release()
        torch.cuda.empty_cache()

        def e2e_step():
            pipe.run(a_pin, b_pin, out_pin, p=args.p)

        e_steps = max(2, min(args.steps, 5))
        for _ in range(2):
            e2e_step()
        barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(e_steps):
            e2e_step()
        torch.cuda.synchronize()
        e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / e_steps
        barrier()
        line["e2e"] = {"value": ops_total / (e_ms * 1e-3), "unit": "diff-ops/s", "ms_per_step": e_ms,
                       "h2d_bytes_per_step": pipe.h2d_bytes, "d2h_bytes_per_step": pipe.d2h_bytes,
                       "steps": e_steps,
                       "note": "kermac_b200.host.HostCdist: pinned host a, b in; this rank's rows of out[N,M] back to "
                               "pinned host; bytes are per rank"}
        del pipe, a_pin, b_pin, out_pin

    # the remaining benchmark configurations, each outside the headline's timed region
    slab = None
    if world > 1:
        cyc.release()
    del a, b, a_dev, b_dev
    torch.cuda.empty_cache()
    if not args.no_also and not args.no_configs:
        args.no_e2e_side = True
        if world == 1:
            also["cfg1 cdist 2048x2048x64 p=2"] = bench_workloads.brief(bench_workloads.cdist_small(args, ctx))
            also["cfg3 cdist batched p=1.3"] = bench_workloads.brief(bench_workloads.cdist_batched(args, ctx))
            also["cfg4 cdist_grad"] = bench_workloads.brief(bench_workloads.grad(args, ctx))
        also["cfg5 kernel_matvec"] = bench_workloads.brief(bench_workloads.matvec(args, ctx))
    if also:
        line["also"] = also

    if rank == 0 and not args.no_cpu:
        from oracle import cpu_baseline
        use_all_host_threads()
        line["cpu_baseline"] = cpu_baseline.time_cdist_slab(a_store, b_store, args.p, rows=args.cpu_rows, repeats=3,
                                                            budget_s=20.0)
    finish(line)


if __name__ == "__main__":
    main()
