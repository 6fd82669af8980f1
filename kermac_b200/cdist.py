"""`cdist`: batched p-norm distance matrix, the headline operator of kermac.

Signature, defaults and exceptions follow src/kermac/cdist.py:9-83 of the reference.
Two reference defects are not reproduced: `skip_epilogue=True` no longer alters the
shared predefined descriptors (cdist.py:65,75 mutate module-level objects), and
`skip_epilogue=True` with a fractional p returns sum_k |b - a|^p instead of raising.
"""
from __future__ import annotations

import torch

from .build_a_kernel import InnerOperator, KernelDescriptor, KernelType, PowerType, run_kernel

__all__ = ["cdist"]


def cdist(
    a: torch.Tensor,
    b: torch.Tensor,
    out: torch.Tensor = None,
    p: float = 2.0,
    skip_epilogue: bool = False,
    try_to_align: bool = False,
    debug=False,
):
    """out[m, n] = (sum_k |b[n, k] - a[m, k]|^p)^(1/p), or the raw sum with `skip_epilogue`.

    In storage terms (the reference README's c-style loop): a[K, M], b[K, N], out[N, M]
    when every tensor is contiguous along m / n.

    Args:
        a: (M, K) or (L, M, K) float32 CUDA tensor, either majorness.
        b: (N, K) or (L, N, K) float32 CUDA tensor, either majorness.
        out: optional (M, N) or (L, M, N) float32 CUDA tensor; allocated as (L, M, N) if None.
        p: norm order; 1.0 and 2.0 take paths without fractional powers.
        skip_epilogue: leave out the final ^(1/p).
        try_to_align: accepted for compatibility; 16-byte staging is automatic.
        debug: print the kernel variant that is launched.

    Raises:
        TypeError: inputs are not float32 torch tensors.
        ValueError: shapes, strides, batch sizes or devices are invalid.
    """
    descriptor, powers = descriptor_for(p, skip_epilogue)
    return run_kernel(descriptor, a, b, out=out, try_to_align=try_to_align, debug=debug, **powers)


def descriptor_for(p: float, skip_epilogue: bool = False):
    """(KernelDescriptor, power keyword arguments of run_kernel) that `cdist` uses for this p.
    A fresh descriptor every time: nothing shared is modified."""
    if p == 1.0:
        return KernelDescriptor(InnerOperator.DIFF, PowerType.ABS, PowerType.NOOP, KernelType.NONE), {}
    if p == 2.0:
        outer = PowerType.NOOP if skip_epilogue else PowerType.SQRT
        return KernelDescriptor(InnerOperator.DIFF, PowerType.SQUARE, outer, KernelType.NONE), {}
    if skip_epilogue:
        return KernelDescriptor(InnerOperator.DIFF, PowerType.POW, PowerType.NOOP, KernelType.NONE), {"inner_p": p}
    return KernelDescriptor(InnerOperator.DIFF, PowerType.POW, PowerType.POW, KernelType.NONE), {"p": p}
