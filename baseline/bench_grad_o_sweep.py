"""cdist_grad at the gradient benchmark shape (K = 30000 contracted, M = 4096, N = 256, seed 3) for
O in {1, 2, 4, 8, 16, 32, 64} channels: kermac_b200 (its FP32 kernel, its tensor-core kernel and what the
automatic choice takes) next to the reference's own kernel on the same GPU.

    python baseline/bench_grad_o_sweep.py

BENCHMARK INFRASTRUCTURE ONLY: nothing in the kermac_b200 package imports this.  CUDA events, a
256 MB write between launches flushes the L2 (its time is subtracted), one JSON object per O.
The reference kernel (baseline/_ref, built by baseline/build_ref_cubin.py) always spends a 32-wide
channel tile (include/p_norm_gradient.cuh:441-448 of the reference), which is why its time does
not depend on O; the reference's TODO.md:3 asks for exactly this sweep.
"""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import kermac_b200 as kermac  # noqa: E402
from baseline import ref_kernels  # noqa: E402


def timed(fn, steps=5, warmup=2):
    flush = torch.empty(64 * 1024 * 1024, device="cuda")

    def flush_only():
        flush.zero_()

    def flush_and_run():
        flush.zero_()
        fn()

    def ms(f):
        for _ in range(warmup):
            f()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            f()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    return ms(flush_and_run) - ms(flush_only)


def main():
    K, M, N = 30000, 4096, 256
    g = torch.Generator().manual_seed(3)
    b = torch.randn(N, K, generator=g).cuda()
    d = torch.randn(N, M, generator=g).cuda()
    a = torch.rand(M, K, generator=g).t().contiguous().cuda()
    for O in (1, 2, 4, 8, 16, 32, 64):
        c = torch.randn(O, K, generator=g).cuda()
        out = torch.empty(1, O, N, M, device="cuda")
        o_ref = torch.empty(O, N, M, device="cuda")
        row = {"O": O}
        for p in (1.0, 1.5, 2.0, 1.7):
            row[f"ours_p{p:g}_ms"] = round(timed(lambda: kermac.cdist_grad(a, b, c, d, out=out, p=p)), 3)
            if O >= 8 and p in (1.0, 1.7):
                for mode in ("fp32", "tensor"):
                    t = timed(lambda: kermac.cdist_grad(a, b, c, d, out=out, p=p, contraction=mode), steps=3, warmup=1)
                    row[f"{mode}_p{p:g}_ms"] = round(t, 3)
            if ref_kernels.available() and p in (1.0, 1.5):
                ref = timed(lambda: ref_kernels.ref_cdist_grad(a, b, c, d, o_ref, p), steps=3, warmup=1)
                row[f"ref_p{p:g}_ms"] = round(ref, 3)
                kermac.cdist_grad(a, b, c, d, out=out, p=p)
                row[f"diff_p{p:g}"] = float((out[0] - o_ref).abs().max() / o_ref.abs().max())
        print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
