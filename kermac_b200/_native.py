"""ctypes binding of libkermac_b200.so (the C-ABI declared in include/kermac_b200.h).

The library holds the AOT-compiled sm_100a kernels; it takes the place of the
reference's NVRTC JIT and LMDB cubin cache (src/kermac/module_cache/module_cache.py).
There is no fallback: if the library is missing every operator raises.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from typing import Optional

ABI_VERSION = 6

# enum values of include/kermac_b200.h
INNER_DIFF, INNER_DOT = 0, 1
POW_NOOP, POW_ABS, POW_SQUARE, POW_SQRT, POW_POW = 0, 1, 2, 3, 4
KERNEL_NONE, KERNEL_LAPLACE, KERNEL_GAUSSIAN = 0, 1, 2
NORM_L1, NORM_L2, NORM_P = 0, 1, 2
VARIANT_AUTO, VARIANT_CPASYNC, VARIANT_TMA = 0, 1, 2

EXPORTED_SYMBOLS = (
    "kermac_b200_build_kernel",
    "kermac_b200_build_tile_count",
    "kermac_b200_cdist_grad",
    "kermac_b200_cdist_grad_scratch_bytes",
    "kermac_b200_cdist_grad_static",
    "kermac_b200_kernel_matvec",
    "kermac_b200_kernel_matvec_scratch_bytes",
    "kermac_b200_describe_variant",
    "kermac_b200_measure_pipe",
    "kermac_b200_device_error_flag",
    "kermac_b200_selftest_wait_expiry",
    "kermac_b200_copy_2d_async",
    "kermac_b200_last_error",
    "kermac_b200_abi_version",
    "kermac_b200_build_id",
)


class KmHyper(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("value", C.c_float), ("batch_stride", C.c_int64)]


class KmBuildArgs(C.Structure):
    _fields_ = [
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("l", C.c_int32),
        ("a", C.c_void_p), ("a_stride_m", C.c_int64), ("a_stride_k", C.c_int64), ("a_stride_l", C.c_int64),
        ("b", C.c_void_p), ("b_stride_n", C.c_int64), ("b_stride_k", C.c_int64), ("b_stride_l", C.c_int64),
        ("out", C.c_void_p), ("out_stride_m", C.c_int64), ("out_stride_n", C.c_int64), ("out_stride_l", C.c_int64),
        ("inner_operator", C.c_int32), ("inner_power", C.c_int32),
        ("outer_power", C.c_int32), ("kernel_type", C.c_int32),
        ("p_inner", KmHyper), ("p_outer", KmHyper), ("bandwidth", KmHyper), ("regularization", KmHyper),
        ("reg_off_x", C.c_int32), ("reg_off_y", C.c_int32),
        ("epsilon", C.c_float),
        ("variant", C.c_int32),
        ("out_multicast", C.c_int32),
        ("symmetry", C.c_int32),
        ("tile_first", C.c_int32),
        ("tile_count", C.c_int32),
    ]


class KmGradArgs(C.Structure):
    _fields_ = [
        ("m", C.c_int32), ("n", C.c_int32), ("o", C.c_int32), ("k", C.c_int32), ("l", C.c_int32),
        ("a", C.c_void_p), ("lda", C.c_int64), ("a_stride_l", C.c_int64),
        ("b", C.c_void_p), ("ldb", C.c_int64), ("b_stride_l", C.c_int64),
        ("c", C.c_void_p), ("ldc", C.c_int64), ("c_stride_l", C.c_int64),
        ("d", C.c_void_p), ("ldd", C.c_int64), ("d_stride_l", C.c_int64),
        ("out", C.c_void_p), ("out_stride_n", C.c_int64), ("out_stride_o", C.c_int64), ("out_stride_l", C.c_int64),
        ("norm_type", C.c_int32),
        ("p", KmHyper),
        ("scratch", C.c_void_p), ("scratch_bytes", C.c_int64),
        ("split_k", C.c_int32),
        ("contraction", C.c_int32),
    ]


class KmMatvecArgs(C.Structure):
    _fields_ = [
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("o", C.c_int32), ("l", C.c_int32),
        ("a", C.c_void_p), ("a_stride_m", C.c_int64), ("a_stride_k", C.c_int64), ("a_stride_l", C.c_int64),
        ("b", C.c_void_p), ("b_stride_n", C.c_int64), ("b_stride_k", C.c_int64), ("b_stride_l", C.c_int64),
        ("c", C.c_void_p), ("ldc", C.c_int64), ("c_stride_l", C.c_int64),
        ("y", C.c_void_p), ("y_stride_n", C.c_int64), ("y_stride_o", C.c_int64), ("y_stride_l", C.c_int64),
        ("inner_operator", C.c_int32), ("inner_power", C.c_int32),
        ("outer_power", C.c_int32), ("kernel_type", C.c_int32),
        ("p_inner", KmHyper), ("p_outer", KmHyper), ("bandwidth", KmHyper),
        ("epsilon", C.c_float),
        ("scratch", C.c_void_p), ("scratch_bytes", C.c_int64),
        ("split_m", C.c_int32),
        ("contraction", C.c_int32),
        ("regularization", KmHyper),
        ("reg_off_x", C.c_int32), ("reg_off_y", C.c_int32),
    ]


class NativeLibraryError(RuntimeError):
    """libkermac_b200.so is missing, unloadable or of the wrong ABI version."""


_lock = threading.Lock()
_lib: Optional[C.CDLL] = None


def library_path() -> str:
    override = os.environ.get("KERMAC_B200_LIB")
    if override:
        return override
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "libkermac_b200.so")


def _declare(lib: C.CDLL) -> None:
    lib.kermac_b200_build_kernel.argtypes = [C.POINTER(KmBuildArgs), C.c_void_p]
    lib.kermac_b200_build_kernel.restype = C.c_int
    lib.kermac_b200_build_tile_count.argtypes = [C.POINTER(KmBuildArgs)]
    lib.kermac_b200_build_tile_count.restype = C.c_int64
    lib.kermac_b200_selftest_wait_expiry.argtypes = [C.c_int32, C.c_void_p]
    lib.kermac_b200_selftest_wait_expiry.restype = C.c_int
    lib.kermac_b200_copy_2d_async.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                              C.c_int32, C.c_void_p]
    lib.kermac_b200_copy_2d_async.restype = C.c_int
    lib.kermac_b200_cdist_grad.argtypes = [C.POINTER(KmGradArgs), C.c_void_p]
    lib.kermac_b200_cdist_grad.restype = C.c_int
    lib.kermac_b200_cdist_grad_scratch_bytes.argtypes = [C.POINTER(KmGradArgs)]
    lib.kermac_b200_cdist_grad_scratch_bytes.restype = C.c_int64
    lib.kermac_b200_cdist_grad_static.argtypes = [C.POINTER(KmGradArgs), C.c_void_p]
    lib.kermac_b200_cdist_grad_static.restype = C.c_int
    lib.kermac_b200_kernel_matvec.argtypes = [C.POINTER(KmMatvecArgs), C.c_void_p]
    lib.kermac_b200_kernel_matvec.restype = C.c_int
    lib.kermac_b200_kernel_matvec_scratch_bytes.argtypes = [C.POINTER(KmMatvecArgs)]
    lib.kermac_b200_kernel_matvec_scratch_bytes.restype = C.c_int64
    lib.kermac_b200_describe_variant.argtypes = [C.POINTER(KmBuildArgs), C.c_char_p, C.c_int32]
    lib.kermac_b200_describe_variant.restype = C.c_int
    lib.kermac_b200_measure_pipe.argtypes = [C.c_int32, C.c_int32, C.POINTER(C.c_double), C.POINTER(C.c_double)]
    lib.kermac_b200_measure_pipe.restype = C.c_int
    lib.kermac_b200_device_error_flag.argtypes = []
    lib.kermac_b200_device_error_flag.restype = C.c_int
    lib.kermac_b200_last_error.argtypes = []
    lib.kermac_b200_last_error.restype = C.c_char_p
    lib.kermac_b200_abi_version.argtypes = []
    lib.kermac_b200_abi_version.restype = C.c_int
    lib.kermac_b200_build_id.argtypes = []
    lib.kermac_b200_build_id.restype = C.c_char_p


def lib() -> C.CDLL:
    """Loads the library once per process (thread safe) and checks its ABI version."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = library_path()
        if not os.path.exists(path):
            raise NativeLibraryError(
                f"{path} not found: build it with `make -C kermac_b200/csrc -j8` "
                "(kermac_b200 has no fallback path)")
        try:
            handle = C.CDLL(path)
        except OSError as exc:
            raise NativeLibraryError(f"cannot load {path}: {exc}") from exc
        missing = [s for s in EXPORTED_SYMBOLS if not hasattr(handle, s)]
        if missing:
            raise NativeLibraryError(f"{path} lacks symbols {missing}")
        _declare(handle)
        got = handle.kermac_b200_abi_version()
        if got != ABI_VERSION:
            raise NativeLibraryError(f"{path} has ABI version {got}, this package needs {ABI_VERSION}")
        _lib = handle
        return handle


def last_error() -> str:
    msg = lib().kermac_b200_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc: int, what: str) -> None:
    """Raises for a non-zero C-ABI return code: ValueError for rejected arguments
    (negative codes), RuntimeError for CUDA errors (positive codes)."""
    if rc == 0:
        return
    msg = last_error()
    if rc < 0:
        raise ValueError(f"{what}: {msg} (code {rc})")
    raise RuntimeError(f"{what}: CUDA error {rc}: {msg}")


def hyper(value) -> KmHyper:
    """A KmHyper from a python float, a 0-dim / 1-element tensor, or a (L,) tensor."""
    import torch
    h = KmHyper()
    if value is None:
        h.ptr, h.value, h.batch_stride = None, 0.0, 0
    elif isinstance(value, torch.Tensor):
        h.ptr = value.data_ptr()
        h.value = 0.0
        h.batch_stride = 0 if (value.dim() == 0 or value.numel() == 1) else value.stride(0)
    else:
        h.ptr, h.value, h.batch_stride = None, float(value), 0
    return h


def launch_build(args: KmBuildArgs, stream_ptr: int) -> None:
    check(lib().kermac_b200_build_kernel(C.byref(args), C.c_void_p(stream_ptr)), "kermac_b200_build_kernel")


def build_tile_count(args: KmBuildArgs) -> int:
    """Number of 128 x 128 output tiles of one batch entry: the range tile_first / tile_count index."""
    n = int(lib().kermac_b200_build_tile_count(C.byref(args)))
    if n < 0:
        check(n, "kermac_b200_build_tile_count")
    return n


def selftest_wait_expiry(tries: int = 1024, stream_ptr: int = 0) -> None:
    """Launches the one-block kernel whose bounded wait runs out on purpose (see the header)."""
    check(lib().kermac_b200_selftest_wait_expiry(int(tries), C.c_void_p(stream_ptr)), "kermac_b200_selftest_wait_expiry")


def copy_2d_async(dst_ptr: int, dst_pitch: int, src_ptr: int, src_pitch: int, row_bytes: int, rows: int,
                  to_host: bool, stream_ptr: int) -> None:
    """Strided 2-D copy between host and device memory on a stream (see the header)."""
    check(lib().kermac_b200_copy_2d_async(C.c_void_p(dst_ptr), dst_pitch, C.c_void_p(src_ptr), src_pitch, row_bytes, rows,
                                          1 if to_host else 0, C.c_void_p(stream_ptr)), "kermac_b200_copy_2d_async")


def launch_grad(args: KmGradArgs, stream_ptr: int) -> None:
    check(lib().kermac_b200_cdist_grad(C.byref(args), C.c_void_p(stream_ptr)), "kermac_b200_cdist_grad")


GRAD_STATIC_SCRATCH_BYTES = 64 << 20


def launch_grad_static(args: KmGradArgs, stream_ptr: int) -> None:
    """cdist_grad whose k-split scratch is the library's built-in array: for callers that
    must not allocate.  Shares one array between all calls; see include/kermac_b200.h."""
    check(lib().kermac_b200_cdist_grad_static(C.byref(args), C.c_void_p(stream_ptr)), "kermac_b200_cdist_grad_static")


def launch_matvec(args: KmMatvecArgs, stream_ptr: int) -> None:
    check(lib().kermac_b200_kernel_matvec(C.byref(args), C.c_void_p(stream_ptr)), "kermac_b200_kernel_matvec")


def describe_build(args: KmBuildArgs) -> str:
    buf = C.create_string_buffer(512)
    check(lib().kermac_b200_describe_variant(C.byref(args), buf, 512), "kermac_b200_describe_variant")
    return buf.value.decode()


def measure_pipe(kind: int, iterations: int = 4096):
    """(operations per second, milliseconds) of one arithmetic pipe microbenchmark."""
    ops, ms = C.c_double(0.0), C.c_double(0.0)
    check(lib().kermac_b200_measure_pipe(kind, iterations, C.byref(ops), C.byref(ms)), "kermac_b200_measure_pipe")
    return ops.value, ms.value


def device_error_flag() -> int:
    return int(lib().kermac_b200_device_error_flag())
