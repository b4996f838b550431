"""The package as a drop-in: user code and the reference's own tests import ``fastgraphcompute``.

Two subprocess runs (the alias publishes the reference's dispatcher op names, so it gets a
process without the reference's op library):

  * tests/dropin_cases.py -- the reference's op names, the low-level search on caller-binned
    input, the module and helper paths, each against the CPU oracle;
  * the CUDA cases of the reference's own test files, UNMODIFIED, read from a checkout of the
    reference ($FGC_REFERENCE_ROOT, else a directory ``reference`` beside this repository);
    skipped where no checkout exists.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

REFERENCE_CUDA_CASES = [
    "test_binned_select_knn.py::TestBinnedSelectKnn::test_large_binned_select_knn_cuda",
    "test_binned_select_knn.py::TestBinnedSelectKnn::test_large_binned_select_knn_cuda_D8",
    "test_binned_select_knn.py::TestBinnedSelectKnn::test_binned_knn_gradient_cuda_K50",
    "test_binned_select_knn.py::TestBinnedSelectKnn::test_binned_knn_gradient_cuda_K10",
    "test_binned_select_knn.py::TestBinnedSelectKnn::test_jit_script_compatibility_cuda",
    "test_bin_by_coordinates.py::TestBinByCoordinates::test_simple_binning_cuda",
    "test_bin_by_coordinates.py::TestBinByCoordinates::test_out_of_bounds_cuda",
    "test_bin_by_coordinates.py::TestBinByCoordinates::test_large_scale_cuda",
    "test_bin_by_coordinates.py::TestBinByCoordinates::test_large_scale_cuda4D",
    "test_bin_by_coordinates.py::TestBinByCoordinates::test_with_wrapper_on_data_cuda",
    "test_index_replacer.py::TestIndexReplacer::test_index_replacer_cuda",
    "test_gnn_ops.py::TestGravNetOp::test_shape_cuda",
    "test_gnn_ops.py::TestGravNetOp::test_jit_script_compatibility",
    "test_oc_helper.py::TestOcHelper::test_oc_helper_matrices_cuda",
    "test_oc_helper.py::TestOcHelper::test_matrices_large_scale_cuda",
    "test_oc_helper.py::TestOcHelper::test_select_with_default_cuda",
    "test_torch_geometric_interface.py",
]


def _env():
    env = dict(os.environ)
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    return env


def reference_root():
    return os.environ.get("FGC_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")


def test_reference_import_path_and_op_names():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "dropin_cases.py")], env=_env(),
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "DROPIN-OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_reference_test_files_unmodified(tmp_path):
    tests_dir = os.path.join(reference_root(), "tests")
    if not os.path.isfile(os.path.join(tests_dir, "test_binned_select_knn.py")):
        pytest.skip("no checkout of the reference (set FGC_REFERENCE_ROOT)")
    # Run from the reference's tests directory (its oc_helper test opens fixtures by relative
    # path); that directory holds no `fastgraphcompute` package, so the import can only resolve
    # to this repository, which leads the module search path.  No cache is written there.
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", "--rootdir", str(tmp_path)]
                       + REFERENCE_CUDA_CASES,
                       env=_env(), cwd=tests_dir, capture_output=True, text=True, timeout=1200)
    tail = r.stdout[-4000:] + r.stderr[-2000:]
    assert r.returncode == 0, tail
    assert " passed" in r.stdout and "failed" not in r.stdout and "skipped" not in r.stdout, tail
