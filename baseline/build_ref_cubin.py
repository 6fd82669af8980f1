"""Compiles the reference's own CUDA kernels, from the sources where they lie in the reference
checkout, into a cubin for sm_100 with NVRTC - the same way the reference's JIT does
(src/kermac/module_cache/module_cache.py:13-51: `#include <kermac.cuh>`, -std=c++17,
-default-device, diag-suppress 64 and 1055, name expressions for the wanted instantiations).

Output: baseline/_ref/kermac_ref_sm100.cubin and baseline/_ref/kermac_ref_names.json (git-ignored;
they travel to the GPU box as built artefacts).  Nothing of the reference's source is copied.

    python baseline/build_ref_cubin.py [/path/to/reference]
"""
import json
import os
import sys

from cuda.bindings import nvrtc

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

BUILD = "cute_build_kernel<InnerOperator::{op},PowerType::{inner},PowerType::{outer},KernelType::{kernel}," \
        "Majorness::{ma},Majorness::{mb},Alignment::{al},Alignment::{al}>"


def build(inner, outer, kernel="NONE", op="DIFF", ma="COL_MAJOR", mb="COL_MAJOR", al="ALIGN_4"):
    return BUILD.format(op=op, inner=inner, outer=outer, kernel=kernel, ma=ma, mb=mb, al=al)


NAMES = {}
for al in ("ALIGN_1", "ALIGN_4"):
    NAMES[f"cdist_p1_{al}"] = build("ABS", "NOOP", al=al)
    NAMES[f"cdist_p2_{al}"] = build("SQUARE", "SQRT", al=al)
    NAMES[f"cdist_pow_{al}"] = build("POW", "POW", al=al)
# the other descriptors and the skipped epilogues (column-major operands, 16-byte copies)
NAMES["l2_raw"] = build("SQUARE", "NOOP")
NAMES["pow_raw"] = build("POW", "NOOP")
NAMES["laplace_l1"] = build("ABS", "NOOP", "LAPLACE")
NAMES["laplace_l2"] = build("SQUARE", "SQRT", "LAPLACE")
NAMES["gaussian_l2sq"] = build("SQUARE", "NOOP", "GAUSSIAN")
NAMES["mma"] = build("NOOP", "NOOP", op="DOT")
# row-major operands (4-byte copies only in the reference)
NAMES["cdist_p2_rowmajor"] = build("SQUARE", "SQRT", ma="ROW_MAJOR", mb="ROW_MAJOR", al="ALIGN_1")
NAMES["cdist_p1_row_col"] = build("ABS", "NOOP", ma="ROW_MAJOR", mb="COL_MAJOR", al="ALIGN_1")
NAMES["grad_L1"] = "cute_norm_kernel_gradient<NormType::L1>"
NAMES["grad_L2"] = "cute_norm_kernel_gradient<NormType::L2>"
NAMES["grad_P"] = "cute_norm_kernel_gradient<NormType::P>"


def check(res, prog=None):
    err = res[0]
    if err != nvrtc.nvrtcResult.NVRTC_SUCCESS:
        log = b""
        if prog is not None:
            _, size = nvrtc.nvrtcGetProgramLogSize(prog)
            log = b" " * size
            nvrtc.nvrtcGetProgramLog(prog, log)
        raise RuntimeError(f"NVRTC error {err}: {log.decode(errors='replace')[-3000:]}")
    return res[1:] if len(res) > 2 else (res[1] if len(res) == 2 else None)


def main():
    here = os.path.dirname(os.path.abspath(__file__))
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
        "KERMAC_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(here)), "reference"))
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    opts = [b"-std=c++17", b"-arch=sm_100", b"-default-device", b"-diag-suppress=64,1055",
            f"-I{ref}/include".encode(), f"-I{ref}/thirdparty/cutlass/include".encode(),
            f"-I{cuda_home}/include".encode()]
    prog = check(nvrtc.nvrtcCreateProgram(b"#include <kermac.cuh>\n", b"kermac_ref.cu", 0, [], []))
    for expr in NAMES.values():
        check(nvrtc.nvrtcAddNameExpression(prog, expr.encode()))
    check(nvrtc.nvrtcCompileProgram(prog, len(opts), opts), prog)
    lowered = {}
    for key, expr in NAMES.items():
        lowered[key] = check(nvrtc.nvrtcGetLoweredName(prog, expr.encode())).decode()
    size = check(nvrtc.nvrtcGetCUBINSize(prog))
    cubin = b" " * size
    check(nvrtc.nvrtcGetCUBIN(prog, cubin))
    os.makedirs(OUT, exist_ok=True)
    with open(os.path.join(OUT, "kermac_ref_sm100.cubin"), "wb") as f:
        f.write(cubin)
    with open(os.path.join(OUT, "kermac_ref_names.json"), "w") as f:
        json.dump({"expressions": NAMES, "lowered": lowered}, f, indent=1)
    print(f"wrote {size} bytes of cubin with {len(lowered)} kernels to {OUT}")


if __name__ == "__main__":
    main()
