"""Source-compatibility stand-in for the reference's JIT module cache
(src/kermac/module_cache/module_cache.py:121-239).

The reference compiles kernels with NVRTC on first use and keeps cubins in an LMDB
database.  Here every kernel is compiled ahead of time into libkermac_b200.so, so the
cache has nothing to compile or store; the class keeps the constructor and the two
methods user code calls.
"""
from __future__ import annotations

from . import _native

__all__ = ["ModuleCache"]


class ModuleCache:
    def __init__(self, debug=False):
        self.debug = debug

    def compile_and_cache_functions(self, device=None, function_names=(), debug=False):
        library = _native.lib()
        if debug or self.debug:
            print(f'(Kermac Debug) nothing to compile, AOT build: {library.kermac_b200_build_id().decode()}')

    def get_function(self, device, function_name, debug=False):
        raise NotImplementedError(
            "kermac_b200 launches AOT kernels through its C-ABI; there are no per-name kernel objects")
