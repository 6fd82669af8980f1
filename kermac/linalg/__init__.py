"""`kermac.linalg`: the reference's cuSOLVER wrappers (solve_cholesky, solve_lu, eigh;
src/kermac/linalg/ of the reference), which this build leaves untouched and does not copy.

On import this package looks for the reference's own `linalg` sources, in the directory named by
KERMAC_LINALG_PATH or in `src/kermac/linalg` under KERMAC_REFERENCE, and runs them as this
package: their relative imports (`from ..common import FillMode`, `from .cholesky import ...`)
then resolve to kermac_b200's helpers and to the reference's files.  They need the `nvmath`
package (nvmath-python).  When either is missing the import fails with an ImportError that says
which; nothing else of `kermac` depends on it.
"""
import os


def _source_dir():
    explicit = os.environ.get("KERMAC_LINALG_PATH")
    if explicit:
        return explicit
    reference = os.environ.get("KERMAC_REFERENCE")
    if reference:
        return os.path.join(reference, "src", "kermac", "linalg")
    return None


def _load():
    try:
        import nvmath  # noqa: F401 - what the reference's linalg imports first
    except ImportError as exc:
        raise ImportError(
            "kermac.linalg wraps cuSOLVER through the `nvmath` package (nvmath-python), which is not installed; "
            "the distance operators of kermac do not need it") from exc
    source = _source_dir()
    init = os.path.join(source, "__init__.py") if source else None
    if not init or not os.path.exists(init):
        raise ImportError(
            "kermac.linalg is not part of kermac_b200: point KERMAC_LINALG_PATH at the reference's "
            "src/kermac/linalg directory (or KERMAC_REFERENCE at its checkout) to use it with this package")
    __path__[:] = [source]                      # noqa: F821 - submodules come from the reference's directory
    with open(init) as f:
        exec(compile(f.read(), init, "exec"), globals())


_load()
