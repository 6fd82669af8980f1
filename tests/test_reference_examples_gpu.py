"""The reference's example scripts for this path (examples/cdist.py, cdist_grad.py, build_a_kernel.py,
broadcast_kernel.py: its usage contract and timing method) run unchanged through `import kermac`.

Like the reference's test files they are run where they lie: from the reference checkout, else from
the byte-for-byte staging copies this repository's build step places under the git-ignored
baseline/_ref/reference_examples/ on machines that have the checkout.  Skipped when neither exists."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _find(name):
    candidates = []
    if os.environ.get("KERMAC_REFERENCE"):
        candidates.append(os.path.join(os.environ["KERMAC_REFERENCE"], "examples", name))
    candidates.append(os.path.join(os.path.dirname(ROOT), "reference", "examples", name))
    candidates.append(os.path.join(ROOT, "baseline", "_ref", "reference_examples", name))
    for path in candidates:
        if os.path.exists(path):
            return path
    return None


CASES = [
    ("cdist.py", ["-m", "700", "-n", "650", "-k", "96", "-l", "2", "-p", "1.3", "--warmup", "1", "--iters", "2"]),
    ("cdist.py", ["-m", "512", "-n", "384", "-k", "64", "-p", "2.0", "-a", "-t", "ntn", "--warmup", "1", "--iters", "1"]),
    ("cdist_grad.py", ["-m", "300", "-n", "96", "-o", "5", "-k", "400", "-l", "2", "-p", "2.0"]),
    ("cdist_grad.py", ["-m", "256", "-n", "64", "-o", "16", "-k", "300", "-l", "1", "-p", "1.0", "--skip_torch_einsum",
                       "--skip_numeric_compare"]),
    ("build_a_kernel.py", ["-m", "600", "-n", "500", "-k", "48", "-a"]),
    ("broadcast_kernel.py", []),
]


@pytest.mark.parametrize("name, argv", CASES)
def test_reference_example_runs_unchanged(name, argv):
    path = _find(name)
    if path is None:
        pytest.skip(f"the reference's examples/{name} is not on this machine")
    env = dict(os.environ)
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    run = subprocess.run([sys.executable, path] + argv, capture_output=True, text=True, env=env, timeout=600)
    assert run.returncode == 0, (run.stdout[-1500:], run.stderr[-3000:])
    assert "nan" not in run.stdout.lower().replace("nan_to_num", "")
