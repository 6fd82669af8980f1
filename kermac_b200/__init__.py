"""kermac_b200: kermac's fused distance operators on NVIDIA B200 (sm_100a).

Drop-in for the hot path of the kermac package: `cdist`, `cdist_grad`, `run_kernel`
with its descriptors and enums, plus the helper names kermac's other modules import
from the package namespace (the reference's star imports, src/kermac/__init__.py:1-4,
expose them).  New here: `kernel_matvec` and the row-sharding helpers in
`kermac_b200.dist`.
"""
from .common import *            # noqa: F401,F403
from .module_cache import *      # noqa: F401,F403
from .build_a_kernel import *    # noqa: F401,F403
from .cdist import *             # noqa: F401,F403
from .cdist_grad import *        # noqa: F401,F403
from .matvec import *            # noqa: F401,F403
from . import dist               # noqa: F401

__version__ = "0.1.0"
