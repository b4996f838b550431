"""The bounds-check build of the library (-DFGC_DEBUG, libfgc_b200_debug.so) on the golden kNN
cases and on clustered data with far outliers: every index the grid build and the search compute
is checked against its array before it is used, a violation sets FGC_STATUS_DEBUG_BOUNDS in the
status word (and the access is skipped), which the Python wrapper turns into an exception.  The
stand-in for a memory checker on machines where none can be run.  Runs in a process of its own
because a process loads one build of the library."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEBUG_LIB = os.path.join(ROOT, "fastgraphcompute_b200", "libfgc_b200_debug.so")


def test_golden_cases_under_the_bounds_check_build():
    if not os.path.exists(DEBUG_LIB):
        pytest.skip("libfgc_b200_debug.so not built (python fastgraphcompute_b200/build.py --debug)")
    env = dict(os.environ)
    env["FGC_B200_LIB"] = DEBUG_LIB
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider",
                        os.path.join(ROOT, "tests", "test_gpu_parity.py"),
                        "-k", "golden or repeated_search or random_configurations"],
                       env=env, cwd=ROOT, capture_output=True, text=True, timeout=1500)
    tail = r.stdout[-3000:] + r.stderr[-2000:]
    assert r.returncode == 0 and " passed" in r.stdout, tail
