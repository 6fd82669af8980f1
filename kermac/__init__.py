"""`kermac`: the reference package's import name, served by kermac_b200.

Code written against the reference (`import kermac; kermac.cdist(...)`,
`kermac.pre_compile_descriptors(...)`, `from kermac import tensor_stats`) runs unchanged:
this package re-exports everything `kermac_b200` exports, which includes the helper names
the reference leaks through its star imports (src/kermac/__init__.py:1-4) and that its
`linalg` module and examples rely on (`tensor_stats`, `FillMode`, `ceil_div`, `CudaTimer`,
`ModuleCache`, ...).  The submodules the reference's own code imports by path
(`kermac.common`, `kermac.build_a_kernel`, `kermac.cdist`, `kermac.cdist_grad`,
`kermac.module_cache`) resolve to the kermac_b200 modules of the same role.

`kermac.linalg` (the cuSOLVER wrappers, src/kermac/linalg/) is not part of this build and is
not copied here: see kermac/linalg/__init__.py, which loads it from the reference's own
sources on `import kermac.linalg`.  Importing `kermac` itself never needs `nvmath`.
"""
import sys

import kermac_b200 as _impl
from kermac_b200 import *                      # noqa: F401,F403
from kermac_b200 import common as _common, build_a_kernel as _build_a_kernel, cdist as _cdist_module
from kermac_b200 import cdist_grad as _cdist_grad_module, module_cache as _module_cache, matvec as _matvec, dist  # noqa: F401

__version__ = _impl.__version__

# `from .common import *` in kermac_b200 binds the functions `cdist` / `cdist_grad` over the
# submodule attributes of the same name, exactly as in the reference; the modules themselves
# stay importable by path.
for _name, _module in (("common", _common), ("build_a_kernel", _build_a_kernel), ("cdist", _cdist_module),
                       ("cdist_grad", _cdist_grad_module), ("module_cache", _module_cache), ("matvec", _matvec),
                       ("dist", dist)):
    sys.modules.setdefault(f"{__name__}.{_name}", _module)
sys.modules.setdefault(f"{__name__}.module_cache.module_cache", _module_cache)
