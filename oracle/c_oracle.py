"""ctypes access to the C restatement of the oracle (oracle/kermac_oracle.c).
TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "_build", "libkermac_oracle.so")
_INNER = {"DIFF": 0, "DOT": 1}
_POWER = {"NOOP": 0, "ABS": 1, "SQUARE": 2, "SQRT": 3, "POW": 4}
_KERNEL = {"NONE": 0, "LAPLACE": 1, "GAUSSIAN": 2}


def build() -> str:
    subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _LIB


def _lib():
    if not os.path.exists(_LIB):
        build()
    lib = C.CDLL(_LIB)
    lib.km_oracle_build.restype = None
    lib.km_oracle_build.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                    C.c_long, C.c_long, C.c_long, C.c_long, C.c_int, C.c_int, C.c_int, C.c_int,
                                    C.c_double, C.c_double, C.c_double, C.c_double, C.c_double, C.c_int, C.c_int]
    lib.km_oracle_grad.restype = None
    lib.km_oracle_grad.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_int, C.c_int, C.c_int, C.c_int, C.c_long, C.c_long, C.c_long, C.c_long,
                                   C.c_double]
    return lib


def build_kernel_c(a: torch.Tensor, b: torch.Tensor, inner_operator="DIFF", inner_power="SQUARE",
                   outer_power="SQRT", kernel_type="NONE", p_inner=0.0, p_outer=0.0, bandwidth=1.0,
                   epsilon=1e-5, regularization=0.0, reg_off_x=0, reg_off_y=0) -> torch.Tensor:
    """float64 (M, N) for 2-D float32 CPU tensors a (M, K), b (N, K) of any strides."""
    a, b = a.detach().cpu(), b.detach().cpu()
    M, K = a.shape
    N = b.shape[0]
    out = np.empty((M, N), dtype=np.float64)
    _lib().km_oracle_build(a.data_ptr(), b.data_ptr(), out.ctypes.data, M, N, K,
                           a.stride(0), a.stride(1), b.stride(0), b.stride(1),
                           _INNER[inner_operator], _POWER[inner_power], _POWER[outer_power], _KERNEL[kernel_type],
                           float(np.float32(p_inner)), float(np.float32(p_outer)), float(np.float32(bandwidth)),
                           float(np.float32(epsilon)), float(np.float32(regularization)), reg_off_x, reg_off_y)
    return torch.from_numpy(out)


def cdist_grad_c(a, b, c, d, p) -> torch.Tensor:
    """float64 (O, N, M) for 2-D float32 CPU tensors with stride 1 in the last dimension."""
    a, b, c, d = (t.detach().cpu() for t in (a, b, c, d))
    K, M = a.shape
    N = b.shape[0]
    O = c.shape[0]
    out = np.empty((O, N, M), dtype=np.float64)
    _lib().km_oracle_grad(a.data_ptr(), b.data_ptr(), c.data_ptr(), d.data_ptr(), out.ctypes.data,
                          M, N, O, K, a.stride(0), b.stride(0), c.stride(0), d.stride(0), float(np.float32(p)))
    return torch.from_numpy(out)
