"""The C-ABI library loads, exports every function include/kermac_b200.h declares, and
rejects bad arguments before touching a device (no compute calls here)."""
import ctypes
import os
import re

import pytest

from kermac_b200 import _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "kermac_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kermac_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_loads_and_reports_abi_version():
    lib = _native.lib()
    assert lib.kermac_b200_abi_version() == _native.ABI_VERSION
    assert b"sm_100a" in lib.kermac_b200_build_id()
    assert b"abi %d " % _native.ABI_VERSION in lib.kermac_b200_build_id()


def test_every_declared_entry_point_is_exported():
    names = _declared_functions()
    assert len(names) >= 10
    handle = ctypes.CDLL(_native.library_path())
    missing = [n for n in names if not hasattr(handle, n)]
    assert not missing, missing
    assert set(names) == set(_native.EXPORTED_SYMBOLS)


def test_struct_sizes_match_the_header_layout():
    # natural alignment of the C structs (int32 x4, then pointer/int64 runs, ...)
    assert ctypes.sizeof(_native.KmHyper) == 24
    assert ctypes.sizeof(_native.KmBuildArgs) == 16 + 3 * 32 + 16 + 4 * 24 + 16 + 8
    assert ctypes.sizeof(_native.KmGradArgs) == 24 + 4 * 24 + 32 + 8 + 24 + 16 + 8
    assert ctypes.sizeof(_native.KmMatvecArgs) == 24 + 2 * 32 + 24 + 32 + 16 + 3 * 24 + 8 + 16 + 8 + 24 + 8


def _build_args(**kw):
    a = _native.KmBuildArgs()
    a.m, a.n, a.k, a.l = 4, 4, 4, 1
    a.a = a.b = a.out = 0x1000
    a.a_stride_m, a.a_stride_k = 4, 1
    a.b_stride_n, a.b_stride_k = 4, 1
    a.out_stride_m, a.out_stride_n = 1, 4
    for k, v in kw.items():
        setattr(a, k, v)
    return a


@pytest.mark.parametrize("kw, code", [
    (dict(m=-1), -2),
    (dict(l=0), -2),
    (dict(a=None), -1),
    (dict(inner_operator=7), -4),
    (dict(outer_power=9), -4),
    (dict(kernel_type=-1), -4),
    (dict(variant=5), -4),
    (dict(out_multicast=2), -4),
    (dict(a_stride_m=3, a_stride_k=2), -3),
    (dict(out_stride_m=2, out_stride_n=3), -3),
    (dict(a_stride_l=-1), -3),
    (dict(variant=_native.VARIANT_TMA), -3),      # row-major operands cannot take the TMA variant
])
def test_build_kernel_rejects_bad_arguments_without_launching(kw, code):
    lib = _native.lib()
    args = _build_args(**kw)
    assert lib.kermac_b200_build_kernel(ctypes.byref(args), None) == code
    assert _native.last_error()
    with pytest.raises(ValueError):
        _native.launch_build(args, 0)


def test_null_argument_blocks():
    lib = _native.lib()
    assert lib.kermac_b200_build_kernel(None, None) == -1
    assert lib.kermac_b200_cdist_grad(None, None) == -1
    assert lib.kermac_b200_kernel_matvec(None, None) == -1
    assert lib.kermac_b200_describe_variant(None, None, 0) == -1


def test_empty_problems_are_no_ops():
    lib = _native.lib()
    assert lib.kermac_b200_build_kernel(ctypes.byref(_build_args(m=0)), None) == 0
    g = _native.KmGradArgs()
    g.l = 1
    assert lib.kermac_b200_cdist_grad(ctypes.byref(g), None) == 0


def test_describe_variant_reports_the_plan():
    args = _build_args(m=300, n=200, k=64, a_stride_m=64, b_stride_n=64, out_stride_n=300)
    text = _native.describe_build(args)
    assert "variant=cpasync" in text and "tiles=3x2" in text and "exchanged=0" in text
    args = _build_args(m=300, n=200, k=64, a_stride_m=64, b_stride_n=64, out_stride_m=200, out_stride_n=1)
    assert "exchanged=1" in _native.describe_build(args) and "tiles=2x3" in _native.describe_build(args)
    col = _build_args(m=256, n=256, k=64, a_stride_m=1, a_stride_k=256, b_stride_n=1, b_stride_k=256, out_stride_n=256,
                      inner_power=_native.POW_SQUARE, outer_power=_native.POW_SQRT)
    assert "variant=tma" in _native.describe_build(col)
    # a and b are the same matrix here and the square is even in the difference: one triangle of tiles
    assert "symmetric=1" in _native.describe_build(col) and "symmetric=0" in text
    col.symmetry = 1
    assert "symmetric=0" in _native.describe_build(col)
    col.symmetry = 0
    col.reg_off_x = 1
    assert "symmetric=0" in _native.describe_build(col)
    col.reg_off_x = 0
    col.b = 0x2000
    assert "symmetric=0" in _native.describe_build(col)
    col.b = col.a
    col.symmetry = 2
    assert _native.lib().kermac_b200_describe_variant(ctypes.byref(col), ctypes.create_string_buffer(64), 64) == -4
    col.symmetry = 0
    col.inner_power = _native.POW_SQRT
    assert "variant=cpasync" in _native.describe_build(col) and "a_vec16=1" in _native.describe_build(col)


def test_grad_rejects_bad_arguments():
    lib = _native.lib()
    g = _native.KmGradArgs()
    g.m, g.n, g.o, g.k, g.l = 8, 8, 2, 8, 1
    g.a = g.b = g.c = g.d = g.out = 0x1000
    g.lda = g.ldd = g.out_stride_n = 8
    g.ldb = g.ldc = 8
    g.out_stride_o = 64
    g.norm_type = 5
    assert lib.kermac_b200_cdist_grad(ctypes.byref(g), None) == -4
    g.norm_type = 0
    g.lda = 4
    assert lib.kermac_b200_cdist_grad(ctypes.byref(g), None) == -3
    g.lda = 8
    g.split_k = 4       # asks for a split without providing scratch: rejected before any launch
    assert lib.kermac_b200_cdist_grad_scratch_bytes(ctypes.byref(g)) == 4 * 8 * 8 * 2 * 4


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("KERMAC_B200_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_native, "_lib", None)
    with pytest.raises(_native.NativeLibraryError):
        _native.lib()
