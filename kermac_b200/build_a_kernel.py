"""`run_kernel` ("build a kernel"): the fused inner-op -> sum over k -> outer-op ->
kernel-function operator of kermac, on AOT-compiled sm_100a kernels.

API, argument meaning, defaults and exceptions follow the reference's
src/kermac/build_a_kernel.py (enums :15-37, KernelDescriptor :39-71, predefined
descriptors :73-119, pre_compile_descriptors :121-156, run_kernel :158-394).
What differs, on purpose:
  * nothing is JIT-compiled: the launch goes through the C-ABI of libkermac_b200.so;
  * float hyper-parameters are passed by value (no device tensor per call);
  * the difference is b - a for every output layout, and the diagonal rule is
    ``regularization_offset_x + m == regularization_offset_y + n`` for every output
    layout (the reference exchanges a and b for row-major outputs without exchanging
    the sign or the offsets, build_a_kernel.py:323-336);
  * `try_to_align` is accepted and ignored: 16-byte staging is chosen automatically
    from the pointers and pitches.
"""
from __future__ import annotations

import os
from enum import Enum, auto
from typing import Any, List, Optional, Union

import numpy as np
import torch

from . import _native
from .common import merge_batch_size, tensor_stats

__all__ = [
    "InnerOperator", "PowerType", "KernelType", "Symmetry", "KernelDescriptor",
    "kernel_descriptor_laplace_l1", "kernel_descriptor_laplace_l2", "kernel_descriptor_p_norm",
    "kernel_descriptor_l1_norm", "kernel_descriptor_l2_norm", "kernel_descriptor_mma",
    "pre_compile_descriptors", "run_kernel",
]


class InnerOperator(Enum):
    DIFF = auto()
    DOT = auto()


class PowerType(Enum):
    NOOP = auto()
    ABS = auto()
    SQUARE = auto()
    SQRT = auto()
    POW = auto()


class KernelType(Enum):
    NONE = auto()
    LAPLACE = auto()
    GAUSSIAN = auto()


class Symmetry(Enum):
    NonSymmetric = auto()
    Symmetric = auto()


_INNER_CODE = {InnerOperator.DIFF: _native.INNER_DIFF, InnerOperator.DOT: _native.INNER_DOT}
_POWER_CODE = {PowerType.NOOP: _native.POW_NOOP, PowerType.ABS: _native.POW_ABS,
               PowerType.SQUARE: _native.POW_SQUARE, PowerType.SQRT: _native.POW_SQRT,
               PowerType.POW: _native.POW_POW}
_KERNEL_CODE = {KernelType.NONE: _native.KERNEL_NONE, KernelType.LAPLACE: _native.KERNEL_LAPLACE,
                KernelType.GAUSSIAN: _native.KERNEL_GAUSSIAN}
_VARIANT_ENV = {"": _native.VARIANT_AUTO, "auto": _native.VARIANT_AUTO,
                "cpasync": _native.VARIANT_CPASYNC, "tma": _native.VARIANT_TMA}


class KernelDescriptor:
    """Which fused operator to run: ``Kfn(outer(sum_k inner(b (-|*) a)))``."""

    def __init__(self, inner_operator, inner_power, outer_power, kernel_type):
        self._inner_operator = inner_operator
        self._inner_power = inner_power
        self._outer_power = outer_power
        self._kernel_type = kernel_type

    def _codes(self):
        try:
            return (_INNER_CODE[self._inner_operator], _POWER_CODE[self._inner_power],
                    _POWER_CODE[self._outer_power], _KERNEL_CODE[self._kernel_type])
        except KeyError as exc:
            raise ValueError(f"KernelDescriptor holds an unknown enum value: {exc}") from None

    def __repr__(self):
        return (f"KernelDescriptor({self._inner_operator.name}, {self._inner_power.name}, "
                f"{self._outer_power.name}, {self._kernel_type.name})")


kernel_descriptor_laplace_l1 = KernelDescriptor(
    inner_operator=InnerOperator.DIFF, inner_power=PowerType.ABS,
    outer_power=PowerType.NOOP, kernel_type=KernelType.LAPLACE)

kernel_descriptor_laplace_l2 = KernelDescriptor(
    inner_operator=InnerOperator.DIFF, inner_power=PowerType.SQUARE,
    outer_power=PowerType.SQRT, kernel_type=KernelType.LAPLACE)

kernel_descriptor_p_norm = KernelDescriptor(
    inner_operator=InnerOperator.DIFF, inner_power=PowerType.POW,
    outer_power=PowerType.POW, kernel_type=KernelType.NONE)

kernel_descriptor_l1_norm = KernelDescriptor(
    inner_operator=InnerOperator.DIFF, inner_power=PowerType.ABS,
    outer_power=PowerType.NOOP, kernel_type=KernelType.NONE)

kernel_descriptor_l2_norm = KernelDescriptor(
    inner_operator=InnerOperator.DIFF, inner_power=PowerType.SQUARE,
    outer_power=PowerType.SQRT, kernel_type=KernelType.NONE)

kernel_descriptor_mma = KernelDescriptor(
    inner_operator=InnerOperator.DOT, inner_power=PowerType.NOOP,
    outer_power=PowerType.NOOP, kernel_type=KernelType.NONE)


def pre_compile_descriptors(device, descriptors: List[Any], try_to_align=False, debug=False):
    """Kept for source compatibility with the JIT-based reference (build_a_kernel.py:121-156).

    Every kernel variant is compiled ahead of time, so this only checks that the
    descriptors are well formed and that the native library loads.
    """
    for descriptor in descriptors:
        descriptor._codes()
    library = _native.lib()
    if debug:
        print(f'(Kermac Debug) AOT kernels already built: {library.kermac_b200_build_id().decode()}')


# --------------------------------------------------------------------------- helpers
def _is_cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


def _current_stream_for(tensor_device):
    """(stream pointer) of torch's current stream, which must live on `tensor_device`."""
    pt_stream = torch.cuda.current_stream()
    if pt_stream.device != tensor_device:
        raise ValueError(
            f"cuda stream must be on the same device as the tensors: got {pt_stream.device}, expected {tensor_device}")
    return pt_stream.cuda_stream


def _check_descriptor_arguments(kd: KernelDescriptor, p, inner_p, outer_p, bandwidth, epsilon, regularization):
    if kd._inner_power is PowerType.POW:
        if p is None and inner_p is None:
            raise ValueError("'inner_power' 'PowerType' is 'Pow' but 'p' and 'inner_p' is not set")
    elif p is not None or inner_p is not None:
        raise ValueError("'inner_power' 'PowerType' is not 'Pow' but 'p' or 'inner_p' is set")
    if kd._outer_power is PowerType.POW:
        if p is None and outer_p is None:
            raise ValueError("'outer_power' 'PowerType' is 'Pow' but 'p' and 'outer_p' is not set")
    elif p is not None or outer_p is not None:
        raise ValueError("'outer_power' 'PowerType' is not 'Pow' but 'p' or 'outer_p' is set")
    if kd._kernel_type is KernelType.NONE:
        if bandwidth is not None or epsilon is not None or regularization is not None:
            raise ValueError("'KernelType' is 'None' but 'bandwidth' or 'epsilon' or 'regularization' is set")
    elif bandwidth is None:
        raise ValueError("'KernelType' is not 'None' but 'bandwidth' is not set")
    if p is not None and inner_p is not None:
        raise ValueError("'p' is not 'None' but 'inner_p' is also not 'None")
    if p is not None and outer_p is not None:
        raise ValueError("'p' is not 'None' but 'outer_p' is also not 'None")


def _check_hyper_tensor(name: str, value, tensor_device):
    if isinstance(value, torch.Tensor):
        if value.dtype != torch.float32:
            raise TypeError(f"`{name}` tensor must have dtype torch.float32")
        if not _is_cuda(value) or value.device != tensor_device:
            raise ValueError(f"`{name}` tensor must be on the same CUDA device as inputs")


def _resolve_powers(p, inner_p, outer_p):
    """(inner, outer) hyper-parameters; `p` sets inner = p and outer = 1 / p in fp32."""
    if p is None:
        return inner_p, outer_p
    if isinstance(p, torch.Tensor):
        inner = p.contiguous()
        return inner, 1.0 / inner
    inner = np.float32(p)
    with np.errstate(divide="ignore"):
        outer = np.float32(1.0) / inner
    return float(inner), float(outer)


def _forced_variant() -> int:
    name = os.environ.get("KERMAC_B200_VARIANT", "").strip().lower()
    if name not in _VARIANT_ENV:
        raise ValueError(f"KERMAC_B200_VARIANT={name!r} is not one of {sorted(k for k in _VARIANT_ENV if k)}")
    return _VARIANT_ENV[name]


def _validate_operands(a, b, out):
    if not isinstance(a, torch.Tensor) or not isinstance(b, torch.Tensor):
        raise TypeError("a and b must be PyTorch tensors")
    if out is not None and not isinstance(out, torch.Tensor):
        raise TypeError("out must be a PyTorch tensor if provided")
    if a.dtype != torch.float32 or b.dtype != torch.float32:
        raise TypeError("a and b must have dtype torch.float32")
    if out is not None and out.dtype != torch.float32:
        raise TypeError("out must have dtype torch.float32")
    if not _is_cuda(a) or not _is_cuda(b):
        raise ValueError("a and b must be on a CUDA device")
    if out is not None and not _is_cuda(out):
        raise ValueError("out must be on a CUDA device")
    if b.device != a.device:
        raise ValueError(f"All inputs must be on the same CUDA device: got {[x.device for x in (a, b)]}")
    if out is not None and out.device != a.device:
        raise ValueError(f"out must be on the same CUDA device as inputs: got {out.device}, expected {a.device}")


def _marshal_build(kernel_descriptor, a, b, out, p, inner_p, outer_p, bandwidth, epsilon, regularization,
                   regularization_offset_x, regularization_offset_y):
    """Validates one run_kernel call and returns (KmBuildArgs, out, keep_alive)."""
    _check_descriptor_arguments(kernel_descriptor, p, inner_p, outer_p, bandwidth, epsilon, regularization)
    if not isinstance(a, torch.Tensor) or not isinstance(b, torch.Tensor):
        raise TypeError("a and b must be PyTorch tensors")
    if out is not None and not isinstance(out, torch.Tensor):
        raise TypeError("out must be a PyTorch tensor if provided")

    L = 1
    for name, value, dims, optional in (
            ('p', p, 0, True), ('inner_p', inner_p, 0, True), ('outer_p', outer_p, 0, True),
            ('bandwidth', bandwidth, 0, True), ('regularization', regularization, 0, True),
            ('a', a, 2, False), ('b', b, 2, False), ('out', out, 2, True)):
        L = merge_batch_size(name, L, value, expected_dims=dims, can_be_none=optional)

    _validate_operands(a, b, out)
    tensor_device = a.device
    stats_a, stats_b = tensor_stats(a), tensor_stats(b)
    _, M, K_a = stats_a.shape
    _, N, K_b = stats_b.shape
    if K_a != K_b:
        raise ValueError(f"K dimensions must match: got {K_a} for a and {K_b} for b")
    K = K_a

    if out is not None:
        L_c = 1 if out.dim() == 2 else out.size(0)
        stats_c = tensor_stats(out)
        _, M_c, N_c = stats_c.shape
        if (M_c, N_c) != (M, N):
            raise ValueError(f"out must have shape (M={M}, N={N}), got {(M_c, N_c)}")
        if L_c != L and L != 1:
            raise ValueError(f"out must have batch dimension (L={L}), got {(L_c)}")
    else:
        out = torch.empty((L, M, N), dtype=torch.float32, device=tensor_device)
        stats_c = tensor_stats(out)

    for name, value in (('inner_p', inner_p), ('outer_p', outer_p), ('p', p),
                        ('bandwidth', bandwidth), ('regularization', regularization)):
        _check_hyper_tensor(name, value, tensor_device)
    inner_p, outer_p = _resolve_powers(p, inner_p, outer_p)

    inner_code, inner_power_code, outer_power_code, kernel_code = kernel_descriptor._codes()
    args = _native.KmBuildArgs()
    args.m, args.n, args.k, args.l = M, N, K, L
    args.a = a.data_ptr()
    args.a_stride_m, args.a_stride_k = stats_a.matrix_strides
    args.a_stride_l = stats_a.batch_stride
    args.b = b.data_ptr()
    args.b_stride_n, args.b_stride_k = stats_b.matrix_strides
    args.b_stride_l = stats_b.batch_stride
    args.out = out.data_ptr()
    args.out_stride_m, args.out_stride_n = stats_c.matrix_strides
    args.out_stride_l = stats_c.batch_stride
    args.inner_operator, args.inner_power = inner_code, inner_power_code
    args.outer_power, args.kernel_type = outer_power_code, kernel_code
    args.p_inner = _native.hyper(inner_p)
    args.p_outer = _native.hyper(outer_p)
    args.bandwidth = _native.hyper(bandwidth)
    args.regularization = _native.hyper(regularization)
    args.reg_off_x = int(regularization_offset_x)
    args.reg_off_y = int(regularization_offset_y)
    args.epsilon = 1e-5 if epsilon is None else float(epsilon)
    args.variant = _forced_variant()
    # symmetric problems (a and b the same view) are computed from one triangle of tiles and
    # mirrored, with identical bits; KERMAC_B200_SYMMETRY=off computes every tile
    args.symmetry = 1 if os.environ.get("KERMAC_B200_SYMMETRY", "auto").strip().lower() == "off" else 0
    keep_alive = (inner_p, outer_p, bandwidth, regularization)
    return args, out, keep_alive


def run_kernel(
    kernel_descriptor: KernelDescriptor,
    a: torch.Tensor,
    b: torch.Tensor,
    out: torch.Tensor = None,
    p: Optional[Union[float, torch.Tensor]] = None,
    inner_p: Optional[Union[float, torch.Tensor]] = None,
    outer_p: Optional[Union[float, torch.Tensor]] = None,
    bandwidth: Optional[Union[float, torch.Tensor]] = None,
    epsilon: Optional[float] = None,
    regularization: Optional[Union[float, torch.Tensor]] = None,
    regularization_offset_x: int = 0,
    regularization_offset_y: int = 0,
    try_to_align: bool = False,
    debug=False,
):
    """out[l, m, n] = Kfn(outer(sum_k inner(b[l, n, k] (-|*) a[l, m, k]))).

    a: (M, K) or (L, M, K); b: (N, K) or (L, N, K); out: (M, N) or (L, M, N); float32 CUDA
    tensors of either majorness, any pitch (views are fine).  Batch extents of a, b and of
    tensor hyper-parameters must be 1 or agree; extent-1 operands broadcast.  When `out`
    is None a (L, M, N) tensor is allocated.  Launches on torch's current stream and
    returns without synchronising.

    The TMA-staged kernels wait on their copies with a bound; if such a wait ever runs out the
    affected tiles are not written and a device flag is raised.  Nothing here reads it: poll
    `kermac_b200._native.device_error_flag()` at your own synchronisation points (0 = clean).
    """
    args, out, keep_alive = _marshal_build(
        kernel_descriptor, a, b, out, p, inner_p, outer_p, bandwidth, epsilon, regularization,
        regularization_offset_x, regularization_offset_y)
    stream_ptr = _current_stream_for(a.device)
    if debug:
        print(f'(Kermac Debug) Launching kernel: {_native.describe_build(args)}')
    _native.launch_build(args, stream_ptr)
    del keep_alive
    return out
