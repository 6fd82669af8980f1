"""Runs the reference's own CUDA kernels (the cubin built by baseline/build_ref_cubin.py) on torch
tensors through the CUDA driver API, so they can be timed and compared on the same GPU.

BENCHMARK / TEST INFRASTRUCTURE ONLY: nothing in the kermac_b200 package imports this.

The launches follow the reference's host code: grid, block and the argument list of
`cute_build_kernel` as packed in src/kermac/build_a_kernel.py:348-390, and of
`cute_norm_kernel_gradient` as packed in src/kermac/cdist_grad.py:200-235.  Only the
COL_MAJOR / COL_MAJOR instantiations are built, so a, b and out must be "column major" in the
reference's sense (first matrix index contiguous), which is the layout of its headline benchmark.
"""
from __future__ import annotations

import ctypes as C
import json
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
CUBIN = os.path.join(HERE, "_ref", "kermac_ref_sm100.cubin")
NAMES = os.path.join(HERE, "_ref", "kermac_ref_names.json")

_state = {}


def available() -> bool:
    return os.path.exists(CUBIN) and os.path.exists(NAMES)


def _driver():
    from cuda.bindings import driver
    return driver


def _check(res):
    err = res[0]
    if int(err) != 0:
        raise RuntimeError(f"CUDA driver error {err}")
    return res[1] if len(res) == 2 else res[1:]


def _function(key: str):
    if "module" not in _state:
        torch.cuda.init()
        torch.zeros(1, device="cuda")                      # makes torch's primary context current
        drv = _driver()
        with open(CUBIN, "rb") as f:
            _state["module"] = _check(drv.cuModuleLoadData(f.read()))
        with open(NAMES) as f:
            names = json.load(f)
        _state["names"], _state["expressions"] = names["lowered"], names["expressions"]
    if key not in _state:
        drv = _driver()
        _state[key] = _check(drv.cuModuleGetFunction(_state["module"], _state["names"][key].encode()))
    return _state[key]


def _col_major_ld(t: torch.Tensor, what: str):
    if t.dim() == 2:
        t = t.unsqueeze(0)
    if t.stride(-2) != 1:
        raise ValueError(f"{what} must have its first matrix index contiguous")
    batch_stride = 0 if t.size(0) == 1 else t.stride(0)
    return t, t.stride(-1), batch_stride


def ref_cdist(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, p: float, aligned: bool = True) -> torch.Tensor:
    """out[l, m, n] = (sum_k |b[l,n,k] - a[l,m,k]|^p)^(1/p) with the reference's kernel."""
    a3, lda, bsa = _col_major_ld(a, "a")
    b3, ldb, bsb = _col_major_ld(b, "b")
    c3, ldc, bsc = _col_major_ld(out, "out")
    L = max(a3.size(0), b3.size(0))
    M, K = a3.shape[-2:]
    N = b3.shape[-2]
    al = "ALIGN_4" if aligned else "ALIGN_1"
    key = {1.0: "cdist_p1_", 2.0: "cdist_p2_"}.get(p, "cdist_pow_") + al
    fn = _function(key)
    if aligned:
        for t, ld, what in ((a3, lda, "a"), (b3, ldb, "b")):
            if t.data_ptr() % 16 != 0 or ld % 4 != 0 or (t.size(0) > 1 and t.stride(0) % 4 != 0):
                raise ValueError(f"{what} is not 16-byte aligned (pointer, pitch or batch stride)")
    dev = a.device
    p_inner = torch.tensor(float(p) if key.startswith("cdist_pow") else 0.0, dtype=torch.float32, device=dev)
    p_outer = 1.0 / p_inner if key.startswith("cdist_pow") else torch.tensor(0.0, dtype=torch.float32, device=dev)
    zero = torch.tensor(0.0, dtype=torch.float32, device=dev)
    values = (M, N, K, L,
              a3.data_ptr(), lda, bsa, b3.data_ptr(), ldb, bsb, c3.data_ptr(), ldc, bsc,
              p_inner.data_ptr(), 0, p_outer.data_ptr(), 0, zero.data_ptr(), 0, zero.data_ptr(), 0,
              0, 0, 1e-5)
    types = (C.c_int32,) * 4 + (C.c_void_p, C.c_uint64, C.c_uint64) * 3 + (C.c_void_p, C.c_uint64) * 4 + \
            (C.c_int32, C.c_int32, C.c_float)
    grid = ((M + 127) // 128, (N + 127) // 128, L)
    stream = torch.cuda.current_stream().cuda_stream
    _check(_driver().cuLaunchKernel(fn, grid[0], grid[1], grid[2], 256, 1, 1, 0, _driver().CUstream(stream), (values, types), 0))
    _state["keep"] = (p_inner, p_outer, zero)
    return out


def _ld(t: torch.Tensor, row_major: bool, what: str):
    if t.dim() == 2:
        t = t.unsqueeze(0)
    if row_major:
        if t.stride(-1) != 1:
            raise ValueError(f"{what} must have its second matrix index contiguous")
        ld = t.stride(-2)
    else:
        if t.stride(-2) != 1:
            raise ValueError(f"{what} must have its first matrix index contiguous")
        ld = t.stride(-1)
    return t, ld, (0 if t.size(0) == 1 else t.stride(0))


def ref_run_kernel(key: str, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, p_inner: float = 0.0,
                   p_outer: float = 0.0, bandwidth: float = 0.0, regularization: float = 0.0, off_x: int = 0,
                   off_y: int = 0, epsilon: float = 1e-5, a_row_major: bool = False, b_row_major: bool = False):
    """Launches the `cute_build_kernel` instantiation built under `key` (see build_ref_cubin.py) with scalar
    hyper-parameters.  `out` must have its first matrix index contiguous (the kernel writes column-major C)."""
    a3, lda, bsa = _ld(a, a_row_major, "a")
    b3, ldb, bsb = _ld(b, b_row_major, "b")
    c3, ldc, bsc = _ld(out, False, "out")
    L = max(a3.size(0), b3.size(0))
    M, K = a3.shape[-2:]
    N = b3.shape[-2]
    fn = _function(key)
    if "ALIGN_4" in _state["expressions"][key]:
        # the 16-byte-copy instantiations fault on anything else (the reference's host code only
        # selects them after the same check, src/kermac/common.py:110-116)
        for t, ld, what in ((a3, lda, "a"), (b3, ldb, "b")):
            if t.data_ptr() % 16 != 0 or ld % 4 != 0 or (t.size(0) > 1 and t.stride(0) % 4 != 0):
                raise ValueError(f"{what} is not 16-byte aligned (pointer, pitch or batch stride) for {key}")
    hyper = torch.tensor([p_inner, p_outer, bandwidth, regularization], dtype=torch.float32, device=a.device)
    hp = hyper.data_ptr()
    values = (M, N, K, L,
              a3.data_ptr(), lda, bsa, b3.data_ptr(), ldb, bsb, c3.data_ptr(), ldc, bsc,
              hp, 0, hp + 4, 0, hp + 8, 0, hp + 12, 0, off_x, off_y, epsilon)
    types = (C.c_int32,) * 4 + (C.c_void_p, C.c_uint64, C.c_uint64) * 3 + (C.c_void_p, C.c_uint64) * 4 + \
            (C.c_int32, C.c_int32, C.c_float)
    grid = ((M + 127) // 128, (N + 127) // 128, L)
    stream = torch.cuda.current_stream().cuda_stream
    _check(_driver().cuLaunchKernel(fn, grid[0], grid[1], grid[2], 256, 1, 1, 0, _driver().CUstream(stream), (values, types), 0))
    _state["keep_hyper"] = hyper
    return out


def ref_cdist_grad(a, b, c, d, out, p: float) -> torch.Tensor:
    """out[o, n, m] = sum_k c[o,k] a[k,m] g(d[n,m] - b[n,k]) with the reference's kernel (2-D operands)."""
    K, M = a.shape
    N, O = b.shape[0], c.shape[0]
    key = {1.0: "grad_L1", 2.0: "grad_L2"}.get(p, "grad_P")
    fn = _function(key)
    p_t = torch.tensor(float(p), dtype=torch.float32, device=a.device)
    blocks_m = (M + 31) // 32
    values = (M, N, O, K, 1, blocks_m,
              a.data_ptr(), a.stride(0), 0, b.data_ptr(), b.stride(0), 0, c.data_ptr(), c.stride(0), 0,
              d.data_ptr(), d.stride(0), 0, out.data_ptr(), out.stride(-2), out.stride(-3), 0,
              p_t.data_ptr(), 0)
    types = (C.c_int32,) * 6 + (C.c_void_p, C.c_uint64, C.c_uint64) * 4 + (C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64) + \
            (C.c_void_p, C.c_uint64)
    grid = (blocks_m, (N + 31) // 32, (O + 31) // 32)
    stream = torch.cuda.current_stream().cuda_stream
    _check(_driver().cuLaunchKernel(fn, grid[0], grid[1], grid[2], 256, 1, 1, 0, _driver().CUstream(stream), (values, types), 0))
    _state["keep_grad"] = p_t
    return out
