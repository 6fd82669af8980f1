"""CPU oracle for the kermac fused-distance operators.  TEST INFRASTRUCTURE ONLY:
nothing in the product package imports this module; tests, the smoke check and the
CPU-baseline leg of the benchmark do.

It restates, in float64 on the host and from the same float32 inputs the GPU sees,
what the reference's kernels define:

  * cdist / run_kernel : the c-style loop of README.md:80-92 and the operator chain of
    include/build_a_kernel.cuh:339-447 (inner operator and power :344-366, outer power
    :374-392, epsilon mask :394-404, Laplace / Gaussian :406-427, diagonal overwrite
    :429-447);
  * cdist_grad         : README.md:122-134 / src/kermac/cdist_grad.py:29-43 and the
    weight of include/p_norm_gradient.cuh:373-394, with sign(x) = copysign(1, x) taken
    from the float32 difference (include/kermac_internal_common.cuh:178-192);
  * kernel_matvec      : run_kernel followed by the coefficient product (no reference
    kernel exists for it; composition of the above).

Hyper-parameter conventions follow src/kermac/build_a_kernel.py: `p` gives
inner_p = float32(p) and outer_p = float32(1) / float32(p) (:281-290); epsilon defaults
to 1e-5 (:375-376).  The difference is always b - a and the diagonal rule is
reg_off_x + m == reg_off_y + n.

Parity pin: the reference ships no CPU implementation, golden vectors or fixtures for
this path; its own tests compare against torch.cdist and a torch.einsum pair at run
time (tests/test_cdist.py:75, tests/test_cdist_grad.py:43-49).  This oracle is pinned
against exactly those two torch formulations in float64 (tests/test_oracle.py and the
fixtures under tests/golden/).  The operator variants the reference never tests
(skip_epilogue, gradient p != 2, Laplace / Gaussian / epsilon / regularisation, DOT)
have no pin on the CPU side beyond this restatement of the kernel source; on a GPU box they are
additionally compared with the reference's own kernels (tests/test_vs_reference_kernels_gpu.py).
Still parity unpinned: batched hyper-parameter tensors and the fused kernel_matvec.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

DIFF, DOT = "DIFF", "DOT"
NOOP, ABS, SQUARE, SQRT, POW = "NOOP", "ABS", "SQUARE", "SQRT", "POW"
NONE, LAPLACE, GAUSSIAN = "NONE", "LAPLACE", "GAUSSIAN"


def _as_batched(t: torch.Tensor, dims: int) -> torch.Tensor:
    """(L?, ...) -> (L, ...) view on the CPU."""
    t = t.detach().cpu()
    return t.unsqueeze(0) if t.dim() == dims else t


def _hyper(value, L: int) -> Optional[torch.Tensor]:
    """float or (L,)/0-dim tensor -> float64 tensor of shape (L,) built from float32 values."""
    if value is None:
        return None
    if isinstance(value, torch.Tensor):
        v = value.detach().cpu().to(torch.float32).reshape(-1)
    else:
        v = torch.tensor([np.float32(value)], dtype=torch.float32)
    if v.numel() == 1:
        v = v.expand(L)
    if v.numel() != L:
        raise ValueError("hyper-parameter batch does not match")
    return v.to(torch.float64)


def _power(x: torch.Tensor, kind: str, p: Optional[float], inner: bool) -> torch.Tensor:
    if kind == NOOP:
        return x
    if kind == ABS:
        return x.abs()
    if kind == SQUARE:
        return x * x
    if kind == SQRT:
        return torch.sqrt(x)
    if kind == POW:
        base = x.abs() if inner else x   # the inner step takes |x| first; the outer one does not
        return torch.pow(base, p)
    raise ValueError(kind)


def build_kernel_ref(a: torch.Tensor, b: torch.Tensor, inner_operator: str = DIFF, inner_power: str = SQUARE,
                     outer_power: str = SQRT, kernel_type: str = NONE, p=None, inner_p=None, outer_p=None,
                     bandwidth=None, epsilon: Optional[float] = None, regularization=None,
                     reg_off_x: int = 0, reg_off_y: int = 0, row_chunk: int = 256) -> torch.Tensor:
    """float64 (L, M, N) result of the fused operator for float32 a (L?, M, K), b (L?, N, K)."""
    a3, b3 = _as_batched(a, 2), _as_batched(b, 2)
    hyper_L = max([1] + [v.numel() for v in (p, inner_p, outer_p, bandwidth, regularization)
                         if isinstance(v, torch.Tensor)])
    L = max(a3.size(0), b3.size(0), hyper_L)
    M, K = a3.shape[-2:]
    N = b3.shape[-2]
    if p is not None:
        pin32 = _hyper(p, L).to(torch.float32)
        inner_pv = pin32.to(torch.float64)
        outer_pv = (torch.tensor(1.0, dtype=torch.float32) / pin32).to(torch.float64)
    else:
        inner_pv, outer_pv = _hyper(inner_p, L), _hyper(outer_p, L)
    bw = _hyper(bandwidth, L)
    reg = _hyper(regularization, L)
    eps = float(np.float32(1e-5 if epsilon is None else epsilon))

    out = torch.empty((L, M, N), dtype=torch.float64)
    for l in range(L):
        al = a3[l if a3.size(0) > 1 else 0].to(torch.float64)
        bl = b3[l if b3.size(0) > 1 else 0].to(torch.float64)
        for m0 in range(0, M, row_chunk):
            am = al[m0:m0 + row_chunk]                     # (m, K)
            if inner_operator == DIFF:
                x = bl.unsqueeze(0) - am.unsqueeze(1)      # (m, N, K) = b[n,k] - a[m,k]
            else:
                x = bl.unsqueeze(0) * am.unsqueeze(1)
            x = _power(x, inner_power, None if inner_pv is None else float(inner_pv[l]), inner=True)
            acc = x.sum(dim=-1)
            acc = _power(acc, outer_power, None if outer_pv is None else float(outer_pv[l]), inner=False)
            if kernel_type != NONE:
                acc = torch.where(acc < eps, torch.zeros_like(acc), acc)
                bwl = float(bw[l])
                gamma = 1.0 / bwl if kernel_type == LAPLACE else 1.0 / (2.0 * bwl * bwl)
                acc = torch.exp(-acc * gamma)
                if reg is not None and float(reg[l]) != 0.0:
                    mm = torch.arange(m0, m0 + am.size(0)).unsqueeze(1) + reg_off_x
                    nn = torch.arange(N).unsqueeze(0) + reg_off_y
                    acc = torch.where(mm == nn, torch.full_like(acc, 1.0 + float(reg[l])), acc)
            out[l, m0:m0 + am.size(0)] = acc
    return out


def cdist_ref(a: torch.Tensor, b: torch.Tensor, p: float = 2.0, skip_epilogue: bool = False,
              row_chunk: int = 256) -> torch.Tensor:
    """float64 (L, M, N): (sum_k |b - a|^p)^(1/p), or the raw sum with skip_epilogue."""
    if p == 1.0:
        return build_kernel_ref(a, b, DIFF, ABS, NOOP, NONE, row_chunk=row_chunk)
    if p == 2.0:
        return build_kernel_ref(a, b, DIFF, SQUARE, NOOP if skip_epilogue else SQRT, NONE, row_chunk=row_chunk)
    if skip_epilogue:
        return build_kernel_ref(a, b, DIFF, POW, NOOP, NONE, inner_p=p, row_chunk=row_chunk)
    return build_kernel_ref(a, b, DIFF, POW, POW, NONE, p=p, row_chunk=row_chunk)


def cdist_grad_ref(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, d: torch.Tensor, p=2.0,
                   n_chunk: int = 16) -> torch.Tensor:
    """float64 (L, O, N, M): sum_k c[o,k] a[k,m] sign(d[n,m]-b[n,k]) |d[n,m]-b[n,k]|^(p-1).

    a (L?, K, M), b (L?, N, K), c (L?, O, K), d (L?, N, M) float32.  The sign comes from
    the float32 difference (an exact tie has a positive sign), the magnitude is float64.
    """
    a3, b3, c3, d3 = (_as_batched(t, 2) for t in (a, b, c, d))
    pL = p.numel() if isinstance(p, torch.Tensor) else 1
    L = max(a3.size(0), b3.size(0), c3.size(0), d3.size(0), pL)
    pv = _hyper(p, L)
    K, M = a3.shape[-2:]
    N = b3.shape[-2]
    O = c3.shape[-2]
    out = torch.empty((L, O, N, M), dtype=torch.float64)
    for l in range(L):
        al, bl, cl, dl = (t[l if t.size(0) > 1 else 0] for t in (a3, b3, c3, d3))
        a64, c64 = al.to(torch.float64), cl.to(torch.float64)
        pl = float(pv[l])
        for n0 in range(0, N, n_chunk):
            dn, bn = dl[n0:n0 + n_chunk], bl[n0:n0 + n_chunk]
            diff32 = dn.unsqueeze(1) - bn.unsqueeze(2)                       # (n, K, M) float32
            sign = torch.copysign(torch.ones_like(diff32), diff32).to(torch.float64)
            mag = (dn.to(torch.float64).unsqueeze(1) - bn.to(torch.float64).unsqueeze(2)).abs()
            if pl == 1.0:
                g = sign
            elif pl == 2.0:
                g = sign * mag
            else:
                g = sign * torch.pow(mag, pl - 1.0)
            w = g * a64.unsqueeze(0)                                          # (n, K, M)
            out[l, :, n0:n0 + dn.size(0)] = torch.einsum('ok,nkm->onm', c64, w)
    return out


def kernel_matvec_ref(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, n_rows: Optional[torch.Tensor] = None,
                      **descriptor) -> torch.Tensor:
    """float64 (L, N, O) (or (L, len(n_rows), O)): sum_m Kmat[m, n] c[o, m]."""
    b3 = _as_batched(b, 2)
    if n_rows is not None:
        b3 = b3[:, n_rows]
    kmat = build_kernel_ref(a, b3, **descriptor)                             # (L, M, N)
    c3 = _as_batched(c, 2).to(torch.float64)
    if c3.size(0) == 1 and kmat.size(0) > 1:
        c3 = c3.expand(kmat.size(0), -1, -1)
    return torch.einsum('lmn,lom->lno', kmat, c3)


# ----------------------------------------------------------------- error metrics
def rel_err_nonneg(x: torch.Tensor, ref: torch.Tensor, tiny: float = 1e-30) -> float:
    """max |x - ref| / max(|ref|, tiny), entries with |ref| < tiny compared absolutely."""
    x = x.detach().cpu().to(torch.float64)
    ref = ref.to(torch.float64)
    err = (x - ref).abs()
    denom = torch.where(ref.abs() < tiny, torch.ones_like(ref), ref.abs())
    return float((err / denom).max()) if err.numel() else 0.0


def rel_err_signed(x: torch.Tensor, ref: torch.Tensor) -> float:
    """max |x - ref| / max |ref| over one output tensor (sums with cancellation)."""
    x = x.detach().cpu().to(torch.float64)
    ref = ref.to(torch.float64)
    if ref.numel() == 0:
        return 0.0
    scale = float(ref.abs().max())
    return float((x - ref).abs().max()) / (scale if scale > 0 else 1.0)
