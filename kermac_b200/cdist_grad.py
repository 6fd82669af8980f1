"""`cdist_grad`: gradient of the p-norm distance, fused with its coefficient contraction.

Signature, argument checks and exceptions follow src/kermac/cdist_grad.py:10-239 of the
reference.  Differences: the batch size of a user-supplied `out` is read from a 4-D
`out` (the reference tests `out.dim() == 2`, which a 3-D/4-D tensor never satisfies),
and when the contracted dimension is long and the output small, the work is split along
k with a scratch buffer taken from torch's caching allocator.
"""
from __future__ import annotations

from typing import Union

import torch

from . import _native
from .build_a_kernel import _current_stream_for, _is_cuda
from .common import merge_batch_size, tensor_stats

__all__ = ["cdist_grad"]


_CONTRACTIONS = {"auto": 0, "fp32": 1, "tensor": 2}   # KM_CONTRACT_* of the C-ABI


def _marshal_grad(a, b, c, d, out, p, contraction="auto"):
    if contraction not in _CONTRACTIONS:
        raise ValueError(f"contraction must be one of {sorted(_CONTRACTIONS)}, got {contraction!r}")
    if not all(isinstance(x, torch.Tensor) for x in (a, b, c, d)):
        raise TypeError("All inputs must be PyTorch tensors")
    if out is not None and not isinstance(out, torch.Tensor):
        raise TypeError("out must be a PyTorch tensor if provided")
    if not all(x.dtype == torch.float32 for x in (a, b, c, d)):
        raise TypeError("All inputs must have dtype torch.float32")
    if out is not None and out.dtype != torch.float32:
        raise TypeError("out must have dtype torch.float32")
    if not all(x.dim() in (2, 3) for x in (a, b, c, d)):
        raise ValueError("All inputs must be 2-dimensional or 3-dimensional with a batch mode")
    if out is not None and out.dim() not in (3, 4):
        raise ValueError("out must be 3-dimensional or 4-dimensional with a batch mode")
    if not all(_is_cuda(x) for x in (a, b, c, d)):
        raise ValueError("All inputs must be on a CUDA device")
    if out is not None and not _is_cuda(out):
        raise ValueError("out must be on a CUDA device")
    tensor_device = a.device
    if not all(x.device == tensor_device for x in (a, b, c, d)):
        raise ValueError(f"All inputs must be on the same CUDA device: got {[x.device for x in (a, b, c, d)]}")
    if out is not None and out.device != tensor_device:
        raise ValueError(f"out must be on the same CUDA device as inputs: got {out.device}, expected {tensor_device}")

    stats = {name: tensor_stats(t) for name, t in (('a', a), ('b', b), ('c', c), ('d', d))}
    _, K, M = stats['a'].shape
    _, N, K_b = stats['b'].shape
    _, O, K_c = stats['c'].shape
    _, N_d, M_d = stats['d'].shape

    L = 1
    L = merge_batch_size('p', L, p, expected_dims=0, can_be_none=False)
    for name, t in (('a', a), ('b', b), ('c', c), ('d', d)):
        L = merge_batch_size(name, L, t, expected_dims=2, can_be_none=False)
    L = merge_batch_size('out', L, out, expected_dims=3, can_be_none=True)
    if out is not None:
        L_e = 1 if out.dim() == 3 else out.size(0)
        if L_e != L and L != 1:
            raise ValueError(f"out must have batch dimension (L={L}), got {(L_e)}")

    if isinstance(p, torch.Tensor):
        if p.dtype != torch.float32:
            raise TypeError("`p` tensor must have dtype torch.float32")
        if not _is_cuda(p) or p.device != tensor_device:
            raise ValueError("`p` tensor must be on the same CUDA device as inputs")

    if (N, K_b) != (N, K):
        raise ValueError(f"Expected shape {(N, K)} for b, got {(N, K_b)}")
    if (O, K_c) != (O, K):
        raise ValueError(f"Expected shape {(O, K)} for c, got {(O, K_c)}")
    if (N_d, M_d) != (N, M):
        raise ValueError(f"Expected shape {(N, M)} for d, got {(N_d, M_d)}")
    if out is not None:
        if L == 1:
            if tuple(out.shape) != (O, N, M) and tuple(out.shape) != (1, O, N, M):
                raise ValueError(f"Expected shape {(O, N, M)} or {(L, O, N, M)} for out, got {out.shape}")
        elif tuple(out.shape) != (L, O, N, M):
            raise ValueError(f"Expected shape {(L, O, N, M)} for out, got {out.shape}")

    for name, t in (('a', a), ('b', b), ('c', c), ('d', d)):
        if t.stride(-1) != 1:
            raise ValueError(f"{name} must have stride 1 in last dimension")
    if out is not None and out.stride(-1) != 1:
        raise ValueError("out must have stride 1 in last dimension")

    if out is None:
        out = torch.empty((L, O, N, M), dtype=torch.float32, device=tensor_device)

    # A python float or a one-element tensor selects the p = 1 / p = 2 kernels; the
    # one-element tensor costs a device-to-host read, as in the reference
    # (cdist_grad.py:181-190).  A (L,) tensor always takes the general kernel.
    p_value = None
    if isinstance(p, torch.Tensor):
        if p.numel() == 1:
            p_value = float(p.item())
    else:
        p_value = float(p)
    if p_value == 1.0:
        norm_type = _native.NORM_L1
    elif p_value == 2.0:
        norm_type = _native.NORM_L2
    else:
        norm_type = _native.NORM_P

    args = _native.KmGradArgs()
    args.m, args.n, args.o, args.k, args.l = M, N, O, K, L
    args.a, args.lda, args.a_stride_l = a.data_ptr(), a.stride(-2), stats['a'].batch_stride
    args.b, args.ldb, args.b_stride_l = b.data_ptr(), b.stride(-2), stats['b'].batch_stride
    args.c, args.ldc, args.c_stride_l = c.data_ptr(), c.stride(-2), stats['c'].batch_stride
    args.d, args.ldd, args.d_stride_l = d.data_ptr(), d.stride(-2), stats['d'].batch_stride
    args.out = out.data_ptr()
    args.out_stride_n, args.out_stride_o = out.stride(-2), out.stride(-3)
    args.out_stride_l = 0 if (L == 1 or out.dim() == 3) else out.stride(-4)
    args.norm_type = norm_type
    args.p = _native.hyper(p if isinstance(p, torch.Tensor) else p_value)
    args.scratch, args.scratch_bytes, args.split_k = None, 0, 0
    args.contraction = _CONTRACTIONS[contraction]
    return args, out


def cdist_grad(
    a: torch.Tensor,           # [K, M]   kernel_matrix
    b: torch.Tensor,           # [N, K]   x
    c: torch.Tensor,           # [O, K]   coefs
    d: torch.Tensor,           # [N, M]   z
    out: torch.Tensor = None,  # [O, N, M] grad
    p: Union[float, torch.Tensor] = 2.0,
    debug=False,
    *,
    contraction: str = "auto",
):
    """out[o, n, m] = sum_k c[o, k] * a[k, m] * sign(d[n, m] - b[n, k]) * |d[n, m] - b[n, k]|^(p - 1).

    Every tensor may carry a leading batch dimension (extent 1 broadcasts) and must have
    stride 1 in its last dimension.  sign() is copysign(1, x): an exact tie counts as +1
    for p = 1, as in the reference's kernel (include/p_norm_gradient.cuh:373-394).

    `contraction` (not in the reference) selects where the products with `c` run: "fp32" as
    packed FP32 FMAs, "tensor" on the tcgen05 tensor cores (three tf32 products per term,
    fp32-level accuracy), "auto" the tensor cores from 17 channels and 256 k on.  The tensor-core
    kernel bounds its waits; one that runs out is reported by
    `kermac_b200._native.device_error_flag()`.

    Raises:
        TypeError: inputs are not float32 torch tensors.
        ValueError: shapes, strides, dimensions or CUDA devices are invalid.
    """
    args, out = _marshal_grad(a, b, c, d, out, p, contraction)
    stream_ptr = _current_stream_for(a.device)
    library = _native.lib()
    import ctypes
    need = int(library.kermac_b200_cdist_grad_scratch_bytes(ctypes.byref(args)))
    scratch = None
    if need > 0:
        scratch = torch.empty(need // 4, dtype=torch.float32, device=a.device)
        args.scratch, args.scratch_bytes = scratch.data_ptr(), need
    if debug:
        print(f'(Kermac Debug) Launching cdist_grad norm_type={args.norm_type} split scratch bytes={need}')
    _native.launch_grad(args, stream_ptr)
    del scratch
    return out
