"""The C-ABI library loads, exports every function include/kermac_b200.h declares, and
rejects bad arguments before touching a device (no compute calls here)."""
import ctypes
import os
import re
import subprocess

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


def _ctypes_layout(cls):
    """{field: (offset, size)} plus the struct size, flattening nothing (nested structs count as one field)."""
    return {name: (getattr(cls, name).offset, getattr(cls, name).size) for name, _ in cls._fields_}, ctypes.sizeof(cls)


def _header_layout(tmp_path):
    """Compiles a C program against include/kermac_b200.h that prints sizeof / offsetof of every field of
    every argument struct, so the Python bindings are compared with what the C compiler lays out."""
    header = open(os.path.join(ROOT, "include", "kermac_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    structs = {}
    for body, name in re.findall(r"typedef struct \w+ \{(.*?)\} (\w+);", header, flags=re.S):
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            # "const float* a", "int64_t a_stride_m, a_stride_k, a_stride_l", "KmHyper p_inner, p_outer"
            names = decl.replace("*", " ").split(None, 1)[1] if not decl.startswith("const") else \
                decl.replace("*", " ").split(None, 2)[2]
            fields += [n.strip() for n in names.split(",")]
        structs[name] = fields
    assert set(structs) == {"KmHyper", "KmBuildArgs", "KmGradArgs", "KmMatvecArgs"}
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "kermac_b200.h"', 'int main(void) {']
    for name, fields in structs.items():
        lines.append(f'  printf("{name} sizeof %zu\\n", sizeof({name}));')
        for f in fields:
            lines.append(f'  printf("{name} {f} %zu %zu\\n", offsetof({name}, {f}), sizeof((({name}*)0)->{f}));')
    lines += ['  printf("abi %d\\n", KERMAC_B200_ABI_VERSION);', '  return 0;', '}']
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)],
                   check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    layout, abi = {}, None
    for line in out.splitlines():
        parts = line.split()
        if parts[0] == "abi":
            abi = int(parts[1])
        elif parts[1] == "sizeof":
            layout.setdefault(parts[0], {})["__sizeof__"] = int(parts[2])
        else:
            layout.setdefault(parts[0], {})[parts[1]] = (int(parts[2]), int(parts[3]))
    return layout, abi


def _assert_matches(header_layout, classes, where):
    for name, cls in classes.items():
        fields, size = _ctypes_layout(cls)
        want = dict(header_layout[name])
        assert size == want.pop("__sizeof__"), f"{where}: sizeof({name})"
        assert list(fields) == list(want), f"{where}: {name} declares {list(fields)}, the header {list(want)}"
        for f, layout in fields.items():
            assert layout == want[f], f"{where}: {name}.{f} is at (offset, size) {layout}, the header says {want[f]}"


def test_bindings_match_the_compiled_header(tmp_path):
    """The ctypes classes of kermac_b200/_native.py against the C compiler's layout of the header."""
    layout, abi = _header_layout(tmp_path)
    assert abi == _native.ABI_VERSION
    _assert_matches(layout, {"KmHyper": _native.KmHyper, "KmBuildArgs": _native.KmBuildArgs,
                             "KmGradArgs": _native.KmGradArgs, "KmMatvecArgs": _native.KmMatvecArgs}, "_native.py")


def test_integration_sample_binding_matches_the_compiled_header(tmp_path):
    """The binding INTEGRATION.md shows a maintainer (its first python block that defines KmBuildArgs) is
    executed as written, minus the library load, and compared the same way."""
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    blocks = [b for b in re.findall(r"```python\n(.*?)```", text, flags=re.S) if "class KmBuildArgs" in b]
    assert len(blocks) == 1
    code = blocks[0]
    assert "kermac_b200_abi_version" in code, "the sample must check the library's ABI version"
    cut = code.index("class KmHyper")
    end = code.index("_lib.kermac_b200_build_kernel.argtypes")
    scope = {}
    exec("import ctypes as C\n" + code[cut:end], scope)
    layout, abi = _header_layout(tmp_path)
    assert f"!= {abi}" in code or f"== {abi}" in code, "the sample must compare with the header's ABI version"
    _assert_matches(layout, {"KmHyper": scope["KmHyper"], "KmBuildArgs": scope["KmBuildArgs"]}, "INTEGRATION.md")


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
    (dict(tile_first=-1), -2),
    (dict(tile_first=2), -2),                     # a 4 x 4 problem has one tile
    (dict(tile_first=0, tile_count=2), -2),
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
    assert "variant=cpasync" in text and "tiles=3x2" in text and "exchanged=0" in text and "tile_range=0+6" in text
    assert _native.build_tile_count(args) == 6
    args.tile_first, args.tile_count = 2, 3
    assert "tile_range=2+3" in _native.describe_build(args) and _native.build_tile_count(args) == 6
    args.tile_first, args.tile_count = 4, 0        # count 0: every tile from tile_first on
    assert "tile_range=4+2" in _native.describe_build(args)
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
    col.out_multicast = 1                          # multicast output: every tile is computed (and sent) by its owner
    assert "symmetric=0" in _native.describe_build(col)
    col.out_multicast = 0
    col.tile_first = 1                             # a partial tile range computes every tile it covers
    assert "symmetric=0" in _native.describe_build(col)
    col.tile_first = 0
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
    g.split_k = 0
    g.contraction = 3   # not a KM_CONTRACT_*
    assert lib.kermac_b200_cdist_grad(ctypes.byref(g), None) == -4
    # the tensor-core form plans its k split for its own tiles (32 x 16 pairs, one block per SM):
    # 2 x 1 tiles of a 64 x 16 output and 4096 k leave room for a split, whichever kernel runs
    g.contraction, g.m, g.n, g.k = 2, 64, 16, 4096
    g.lda = g.ldd = g.out_stride_n = 64
    g.ldb = g.ldc = 4096
    g.out_stride_o = 64 * 16
    assert lib.kermac_b200_cdist_grad_scratch_bytes(ctypes.byref(g)) % (64 * 16 * 2 * 4) == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("KERMAC_B200_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_native, "_lib", None)
    with pytest.raises(_native.NativeLibraryError):
        _native.lib()
