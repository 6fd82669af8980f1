"""`kernel_matvec`: y = K(b, a) @ c^T without ever storing the kernel matrix K.

Additive to the reference API.  It fuses what reference users write as
``run_kernel(descriptor, a, b, ...)`` (src/kermac/build_a_kernel.py:158-394) followed
by a matrix product with coefficients (examples/linalg.py:55-119), which cannot be done
there once M x N no longer fits in memory.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Union

import torch

from . import _native
from .build_a_kernel import (KernelDescriptor, _check_descriptor_arguments, _check_hyper_tensor,
                             _current_stream_for, _is_cuda, _resolve_powers)
from .common import merge_batch_size, tensor_stats

__all__ = ["kernel_matvec"]


def _marshal_matvec(kernel_descriptor, a, b, c, out, p, inner_p, outer_p, bandwidth, epsilon, regularization=None,
                    regularization_offset_x=0, regularization_offset_y=0):
    _check_descriptor_arguments(kernel_descriptor, p, inner_p, outer_p, bandwidth, epsilon, regularization)
    for name, t in (('a', a), ('b', b), ('c', c)):
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{name} must be a PyTorch tensor")
        if t.dtype != torch.float32:
            raise TypeError(f"{name} must have dtype torch.float32")
        if not _is_cuda(t):
            raise ValueError(f"{name} must be on a CUDA device")
        if t.device != a.device:
            raise ValueError("All inputs must be on the same CUDA device")
    if out is not None:
        if not isinstance(out, torch.Tensor):
            raise TypeError("out must be a PyTorch tensor if provided")
        if out.dtype != torch.float32:
            raise TypeError("out must have dtype torch.float32")
        if not _is_cuda(out) or out.device != a.device:
            raise ValueError("out must be on the same CUDA device as inputs")

    L = 1
    for name, value, dims, optional in (
            ('p', p, 0, True), ('inner_p', inner_p, 0, True), ('outer_p', outer_p, 0, True),
            ('bandwidth', bandwidth, 0, True), ('regularization', regularization, 0, True),
            ('a', a, 2, False), ('b', b, 2, False), ('c', c, 2, False), ('out', out, 2, True)):
        L = merge_batch_size(name, L, value, expected_dims=dims, can_be_none=optional)

    stats_a, stats_b, stats_c = tensor_stats(a), tensor_stats(b), tensor_stats(c)
    _, M, K = stats_a.shape
    _, N, K_b = stats_b.shape
    _, O, M_c = stats_c.shape
    if K != K_b:
        raise ValueError(f"K dimensions must match: got {K} for a and {K_b} for b")
    if M_c != M:
        raise ValueError(f"c must have shape (O, M={M}), got {(O, M_c)}")
    if c.stride(-1) != 1:
        raise ValueError("c must have stride 1 in last dimension")
    if out is not None:
        if tuple(out.shape[-2:]) != (N, O):
            raise ValueError(f"out must have shape (N={N}, O={O}), got {tuple(out.shape[-2:])}")
        L_y = 1 if out.dim() == 2 else out.size(0)
        if L_y != L and L != 1:
            raise ValueError(f"out must have batch dimension (L={L}), got {(L_y)}")
    else:
        out = torch.empty((L, N, O), dtype=torch.float32, device=a.device)

    for name, value in (('inner_p', inner_p), ('outer_p', outer_p), ('p', p), ('bandwidth', bandwidth),
                        ('regularization', regularization)):
        _check_hyper_tensor(name, value, a.device)
    inner_p, outer_p = _resolve_powers(p, inner_p, outer_p)

    inner_code, inner_power_code, outer_power_code, kernel_code = kernel_descriptor._codes()
    args = _native.KmMatvecArgs()
    args.m, args.n, args.k, args.o, args.l = M, N, K, O, L
    args.a = a.data_ptr()
    args.a_stride_m, args.a_stride_k = stats_a.matrix_strides
    args.a_stride_l = stats_a.batch_stride
    args.b = b.data_ptr()
    args.b_stride_n, args.b_stride_k = stats_b.matrix_strides
    args.b_stride_l = stats_b.batch_stride
    args.c, args.ldc, args.c_stride_l = c.data_ptr(), c.stride(-2), stats_c.batch_stride
    args.y = out.data_ptr()
    args.y_stride_n, args.y_stride_o = out.stride(-2), out.stride(-1)
    args.y_stride_l = 0 if (out.dim() == 2 or out.size(0) == 1) else out.stride(0)
    args.inner_operator, args.inner_power = inner_code, inner_power_code
    args.outer_power, args.kernel_type = outer_power_code, kernel_code
    args.p_inner = _native.hyper(inner_p)
    args.p_outer = _native.hyper(outer_p)
    args.bandwidth = _native.hyper(bandwidth)
    args.epsilon = 1e-5 if epsilon is None else float(epsilon)
    args.regularization = _native.hyper(regularization)
    args.reg_off_x = int(regularization_offset_x)
    args.reg_off_y = int(regularization_offset_y)
    args.scratch, args.scratch_bytes, args.split_m = None, 0, 0
    return args, out, (inner_p, outer_p, bandwidth, regularization)


_CONTRACTIONS = {"auto": 0, "fp32": 1, "tensor": 2}


def _contraction_code(name: Optional[str]) -> int:
    if name is None:
        name = os.environ.get("KERMAC_B200_CONTRACTION", "auto")
    try:
        return _CONTRACTIONS[str(name).lower()]
    except KeyError:
        raise ValueError(f"contraction must be one of {sorted(_CONTRACTIONS)}, got {name!r}") from None


def kernel_matvec(
    kernel_descriptor: KernelDescriptor,
    a: torch.Tensor,
    b: torch.Tensor,
    c: torch.Tensor,
    out: torch.Tensor = None,
    p: Optional[Union[float, torch.Tensor]] = None,
    inner_p: Optional[Union[float, torch.Tensor]] = None,
    outer_p: Optional[Union[float, torch.Tensor]] = None,
    bandwidth: Optional[Union[float, torch.Tensor]] = None,
    epsilon: Optional[float] = None,
    regularization: Optional[Union[float, torch.Tensor]] = None,
    regularization_offset_x: int = 0,
    regularization_offset_y: int = 0,
    split_m: int = 0,
    contraction: Optional[str] = None,
    debug=False,
):
    """y[l, n, o] = sum_m Kmat[l, m, n] * c[l, o, m], Kmat = run_kernel(kernel_descriptor, a, b, ...).

    a: (M, K) / (L, M, K); b: (N, K) / (L, N, K); c: (O, M) / (L, O, M) with stride 1 along
    m; out: (N, O) / (L, N, O), allocated as (L, N, O) when None.  Hyper-parameters as in
    `run_kernel`, including the diagonal rule: where regularization_offset_x + m ==
    regularization_offset_y + n the kernel value is 1 + regularization, so a square K(X, X)
    gives (K + lambda I) c in one pass.  `split_m` > 1 divides the sum over m
    among that many thread blocks per row tile (0 picks automatically); partial sums are
    added in a fixed order, so the result does not depend on scheduling.  `contraction`
    selects where the coefficient product runs: "tensor" (tcgen05 tensor cores, three tf32
    products per term, fp32-level accuracy), "fp32" (packed FP32 FMAs) or "auto" / None
    (the environment variable KERMAC_B200_CONTRACTION, else the library default: tensor).

    The tensor-core kernel waits on its copies and on the tensor cores with a bound; a wait that
    runs out leaves the affected rows unwritten and raises a device flag that nothing here reads:
    poll `kermac_b200._native.device_error_flag()` at your own synchronisation points.
    """
    args, out, keep_alive = _marshal_matvec(kernel_descriptor, a, b, c, out, p, inner_p, outer_p, bandwidth, epsilon,
                                            regularization, regularization_offset_x, regularization_offset_y)
    stream_ptr = _current_stream_for(a.device)
    args.split_m = int(split_m)
    args.contraction = _contraction_code(contraction)
    need = int(_native.lib().kermac_b200_kernel_matvec_scratch_bytes(ctypes.byref(args)))
    scratch = None
    if need > 0:
        scratch = torch.empty(need // 4, dtype=torch.float32, device=a.device)
        args.scratch, args.scratch_bytes = scratch.data_ptr(), need
    if debug:
        print(f'(Kermac Debug) Launching kernel_matvec split scratch bytes={need}')
    _native.launch_matvec(args, stream_ptr)
    del scratch, keep_alive
    return out
