"""The package under the reference's import name: `import kermac` serves kermac_b200, the helper names
the reference's other modules import are there, `kermac.linalg` fails with a clear ImportError where its
dependency is missing, and the wheel carries both packages and the native library."""
import importlib
import os
import shutil
import subprocess
import sys
import zipfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_kermac_reexports_the_reference_surface():
    import kermac
    import kermac_b200
    # the names the reference lists (src/kermac/__init__.py:6-22) ...
    for name in ("cdist", "cdist_grad", "KernelDescriptor", "run_kernel", "PowerType", "InnerOperator", "KernelType",
                 "Symmetry", "kernel_descriptor_laplace_l1", "kernel_descriptor_laplace_l2", "kernel_descriptor_p_norm",
                 "kernel_descriptor_l1_norm", "kernel_descriptor_l2_norm", "kernel_descriptor_mma",
                 "pre_compile_descriptors"):
        assert getattr(kermac, name) is getattr(kermac_b200, name), name
    # ... and the ones its star imports leak, which linalg and the examples use
    for name in ("tensor_stats", "TensorStats", "FillMode", "Majorness", "Alignment", "ceil_div", "merge_batch_size",
                 "CudaTimer", "PyTorchStreamWrapper", "ModuleCache", "kernel_matvec"):
        assert getattr(kermac, name) is getattr(kermac_b200, name), name
    assert callable(kermac.cdist) and callable(kermac.cdist_grad)


def test_submodules_the_reference_imports_by_path():
    common = importlib.import_module("kermac.common")
    assert common.FillMode is importlib.import_module("kermac_b200.common").FillMode
    assert importlib.import_module("kermac.build_a_kernel").run_kernel is importlib.import_module("kermac").run_kernel
    assert importlib.import_module("kermac.module_cache.module_cache").ModuleCache is importlib.import_module("kermac").ModuleCache


def test_pre_compile_descriptors_keeps_the_reference_signature():
    import kermac
    import torch
    # tests/test_cdist.py:26-31 of the reference calls it like this in setUp
    kermac.pre_compile_descriptors(device=torch.device("cpu"),
                                   descriptors=[kermac.kernel_descriptor_l1_norm, kermac.kernel_descriptor_l2_norm,
                                                kermac.kernel_descriptor_p_norm], try_to_align=True, debug=False)


def test_linalg_import_says_what_is_missing(monkeypatch):
    sys.modules.pop("kermac.linalg", None)
    try:
        import nvmath  # noqa: F401
        have_nvmath = True
    except ImportError:
        have_nvmath = False
    monkeypatch.delenv("KERMAC_LINALG_PATH", raising=False)
    monkeypatch.delenv("KERMAC_REFERENCE", raising=False)
    with pytest.raises(ImportError) as info:
        importlib.import_module("kermac.linalg")
    assert ("KERMAC_LINALG_PATH" if have_nvmath else "nvmath") in str(info.value)
    sys.modules.pop("kermac.linalg", None)
    import kermac                      # the failed import leaves the package usable
    assert callable(kermac.cdist)


def test_wheel_carries_both_packages_and_the_library(tmp_path):
    """pip wheel from a scratch copy of the sources (prebuilt objects travel with their time stamps, so
    make has nothing to redo), then import from the unpacked wheel in a fresh interpreter."""
    src = tmp_path / "src"
    src.mkdir()
    for name in ("pyproject.toml", "setup.py"):
        shutil.copy2(os.path.join(ROOT, name), src / name)
    for name in ("kermac", "kermac_b200", "include"):
        shutil.copytree(os.path.join(ROOT, name), src / name, copy_function=shutil.copy2,
                        ignore=shutil.ignore_patterns("__pycache__"))
    wheels = tmp_path / "wheels"
    res = subprocess.run([sys.executable, "-m", "pip", "wheel", "--no-deps", "--no-build-isolation", "--no-index",
                          "-w", str(wheels), str(src)], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    built = [f for f in os.listdir(wheels) if f.endswith(".whl")]
    assert len(built) == 1 and "linux" in built[0]
    site = tmp_path / "site"
    with zipfile.ZipFile(wheels / built[0]) as z:
        names = [n.split("purelib/")[-1].split("platlib/")[-1] for n in z.namelist()]
    assert "kermac_b200/libkermac_b200.so" in names
    assert "kermac/__init__.py" in names and "kermac/linalg/__init__.py" in names
    assert not any(n.startswith("kermac_b200/csrc") for n in names)
    res = subprocess.run([sys.executable, "-m", "pip", "install", "--no-deps", "--no-index", "--target", str(site),
                          str(wheels / built[0])], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    code = ("import kermac, kermac_b200, os; from kermac_b200 import _native; "
            "assert os.path.dirname(kermac.__file__).startswith(%r); "
            "assert _native.library_path().startswith(%r); "
            "assert _native.lib().kermac_b200_abi_version() == _native.ABI_VERSION; "
            "assert kermac.cdist is kermac_b200.cdist; print('ok')" % (str(site), str(site)))
    env = {k: v for k, v in os.environ.items() if k not in ("PYTHONPATH", "KERMAC_B200_LIB")}
    env["PYTHONPATH"] = str(site)
    run = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=str(tmp_path))
    assert run.returncode == 0 and "ok" in run.stdout, run.stdout + run.stderr


def test_linalg_loads_from_an_external_source_directory(monkeypatch, tmp_path):
    """The mechanism `import kermac.linalg` uses, with stand-ins for what this machine lacks: a fake
    `nvmath` module and a two-file package that imports the way the reference's linalg does
    (`import nvmath`, `from ..common import FillMode`, `from .sub import f`, `import kermac`)."""
    import types
    src = tmp_path / "linalg_src"
    src.mkdir()
    (src / "__init__.py").write_text("from .solver import solve\nall = ['solve']\n")
    (src / "solver.py").write_text(
        "import nvmath\nimport kermac\nfrom ..common import FillMode\n"
        "def solve():\n    return (nvmath.MARK, FillMode.UPPER, kermac.ceil_div(7, 2))\n")
    fake = types.ModuleType("nvmath")
    fake.MARK = "fake-nvmath"
    monkeypatch.setitem(sys.modules, "nvmath", fake)
    monkeypatch.setenv("KERMAC_LINALG_PATH", str(src))
    for name in [n for n in sys.modules if n.startswith("kermac.linalg")]:
        sys.modules.pop(name)
    try:
        linalg = importlib.import_module("kermac.linalg")
        import kermac
        assert linalg.solve() == ("fake-nvmath", kermac.FillMode.UPPER, 4)
        assert kermac.linalg is linalg
        assert importlib.import_module("kermac.linalg.solver").solve is linalg.solve
    finally:
        for name in [n for n in sys.modules if n.startswith("kermac.linalg")]:
            sys.modules.pop(name)
        import kermac
        kermac.__dict__.pop("linalg", None)
