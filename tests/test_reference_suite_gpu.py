"""Runs the reference's own GPU test files for this path, unchanged, against this package through
`import kermac`: tests/test_cdist.py (48 layout / p / alignment combinations against torch.cdist) and
tests/test_cdist_grad.py (p = 2 against the einsum pair) of the reference.

The files are loaded where they lie: from the reference checkout (KERMAC_REFERENCE, or a `reference`
directory beside this repository), else from the byte-for-byte staging copy that this repository's
build step places under the git-ignored baseline/_ref/reference_tests/ on machines that have the
checkout, so that the GPU machine, which has none, can run them.  Nothing of them is part of this
repository.  Skipped when neither exists."""
import importlib.util
import os
import unittest

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _find(name):
    candidates = []
    if os.environ.get("KERMAC_REFERENCE"):
        candidates.append(os.path.join(os.environ["KERMAC_REFERENCE"], "tests", name))
    candidates.append(os.path.join(os.path.dirname(ROOT), "reference", "tests", name))
    candidates.append(os.path.join(ROOT, "baseline", "_ref", "reference_tests", name))
    for path in candidates:
        if os.path.exists(path):
            return path
    return None


@pytest.mark.parametrize("name", ["test_cdist.py", "test_cdist_grad.py"])
def test_reference_test_file_passes_unchanged(name):
    path = _find(name)
    if path is None:
        pytest.skip(f"the reference's tests/{name} is not on this machine")
    import kermac                                        # noqa: F401 - what the file's `import kermac` resolves to
    assert "kermac_b200" in kermac.cdist.__module__
    spec = importlib.util.spec_from_file_location("reference_" + name[:-3], path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    suite = unittest.defaultTestLoader.loadTestsFromModule(module)
    assert suite.countTestCases() >= 1
    result = unittest.TextTestRunner(verbosity=0).run(suite)
    problems = [str(t) + "\n" + tb for t, tb in result.failures + result.errors]
    assert result.wasSuccessful(), "\n".join(problems)[-4000:]
    assert result.testsRun >= 1 and not result.skipped
