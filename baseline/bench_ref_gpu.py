"""Times the reference's own kernels (NVRTC-built for sm_100, baseline/build_ref_cubin.py) next to
kermac_b200 on the same GPU and the same inputs, and reports how far the two results are apart.

    python baseline/bench_ref_gpu.py [--small]

Prints one JSON object per measurement.  Needs baseline/_ref/ (built where the reference checkout
is available) and a B200.
"""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

import kermac_b200 as kermac  # noqa: E402
from baseline import ref_kernels  # noqa: E402


def timed(fn, steps=5, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def max_rel(x, y):
    return float(((x - y).abs() / y.abs().clamp_min(1e-30)).max())


def main():
    if not ref_kernels.available():
        print(json.dumps({"unavailable": "baseline/_ref cubin not built"}))
        return
    small = "--small" in sys.argv
    M = N = 4096 if small else 30000
    K = 256 if small else 1024
    g = torch.Generator().manual_seed(1)
    a = torch.randn(K, M, generator=g).cuda().t()
    b = torch.randn(K, N, generator=g).cuda().t()
    out_ref = torch.empty(N, M, device="cuda").t()
    out_new = torch.empty(N, M, device="cuda").t()
    for p in (1.0, 2.0, 1.3):
        t_new = timed(lambda: kermac.cdist(a, b, out=out_new, p=p))
        for aligned in (True, False):
            t_ref = timed(lambda: ref_kernels.ref_cdist(a, b, out_ref, p, aligned=aligned), steps=3, warmup=1)
            print(json.dumps({"op": "cdist", "M": M, "N": N, "K": K, "p": p,
                              "reference_kernel": "ALIGN_4 (try_to_align=True)" if aligned else "ALIGN_1 (default)",
                              "reference_ms": t_ref, "kermac_b200_ms": t_new, "speedup": t_ref / t_new,
                              "max_rel_diff": max_rel(out_new, out_ref)}), flush=True)
    del out_ref, out_new
    # gradient configuration (operator naming): K contracted
    K, M, N, O = (3000 if small else 30000), 4096, 256, 4
    bb = torch.randn(N, K, generator=g).cuda()
    d = torch.randn(N, M, generator=g).cuda()
    c = torch.randn(O, K, generator=g).cuda()
    aa = torch.rand(K, M, generator=g).cuda()
    o_ref = torch.empty(O, N, M, device="cuda")
    o_new = torch.empty(1, O, N, M, device="cuda")
    for p in (1.0, 1.5):
        t_new = timed(lambda: kermac.cdist_grad(aa, bb, c, d, out=o_new, p=p))
        t_ref = timed(lambda: ref_kernels.ref_cdist_grad(aa, bb, c, d, o_ref, p), steps=3, warmup=1)
        scale = float(o_ref.abs().max())
        print(json.dumps({"op": "cdist_grad", "K": K, "M": M, "N": N, "O": O, "p": p, "reference_ms": t_ref,
                          "kermac_b200_ms": t_new, "speedup": t_ref / t_new,
                          "max_abs_diff_over_max": float((o_new[0] - o_ref).abs().max()) / scale}), flush=True)


if __name__ == "__main__":
    main()
