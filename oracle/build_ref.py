"""TEST INFRASTRUCTURE ONLY: build the reference's own CPU ops into oracle/_ref/.

The reference's CPU implementation of the hot path (binning, binned kNN forward,
kNN gradient, index_replacer and the autograd orchestrator) lives in nine .cpp
files (source list: setup.py:91-101 of the reference).  This script compiles
them with g++ directly *from where they lie* in the reference checkout -- no
source is copied -- together with oracle/ref_cuda_stubs.cpp, and links one
shared object, oracle/_ref/binned_knn_ops.so, against the installed libtorch.

Flags follow the reference (-O2, no -march=native, no fast-math), so x86-64
baseline code without FMA contraction is generated and squared distances keep
the sub/mul/add rounding sequence of binned_select_knn_cpu.cpp:10-19.

Usage:  python oracle/build_ref.py [--reference /path/to/FastGraphCompute]
The output directory is git-ignored; the built .so is loaded with
torch.ops.load_library by oracle/ref_ops.py.
"""
import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT_SO = os.path.join(OUT_DIR, "binned_knn_ops.so")
# single-file op libraries of the loss-side helpers (setup.py:139-159 of the reference)
EXTRA_LIBS = {"oc_helper_cpu.so": ["oc_helper_cpu.cpp"], "oc_helper_helper.so": ["oc_helper_helper.cpp"],
              # brute-force kNN (setup.py:116-129); its CUDA twin is replaced by a stub
              "select_knn_lib.so": ["select_knn.cpp", "select_knn_cpu.cpp", "@ref_cuda_stubs.cpp"]}

CPU_SOURCES = [
    "binned_knn_autograd_kernel.cpp",
    "binned_select_knn.cpp",
    "binned_select_knn_cpu.cpp",
    "bin_by_coordinates.cpp",
    "bin_by_coordinates_cpu.cpp",
    "index_replacer.cpp",
    "index_replacer_cpu.cpp",
    "binned_select_knn_grad.cpp",
    "binned_select_knn_grad_cpu.cpp",
]


def default_reference_root():
    """Checkout of the reference: $FGC_REFERENCE_ROOT, else a directory named ``reference``
    beside this repository."""
    return os.environ.get("FGC_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(reference_root=None, force=False, verbose=True):
    """Compile and link; returns the path of the .so or None if the reference is absent."""
    reference_root = reference_root or default_reference_root()
    ext_dir = os.path.join(reference_root, "fastgraphcompute", "extensions")
    if not os.path.isdir(ext_dir):
        return None
    srcs = [os.path.join(ext_dir, s) for s in CPU_SOURCES]
    srcs.append(os.path.join(HERE, "ref_cuda_stubs.cpp"))
    targets = {OUT_SO: srcs}
    for name, files in EXTRA_LIBS.items():
        targets[os.path.join(OUT_DIR, name)] = [os.path.join(HERE, f[1:]) if f.startswith("@")
                                                else os.path.join(ext_dir, f) for f in files]
    stale = {so: ss for so, ss in targets.items()
             if force or not os.path.exists(so) or any(os.path.getmtime(so) < os.path.getmtime(x) for x in ss)}
    if not stale:
        return OUT_SO

    import torch
    from torch.utils import cpp_extension

    os.makedirs(OUT_DIR, exist_ok=True)
    obj_dir = os.path.join(OUT_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    inc = []
    for p in cpp_extension.include_paths():
        inc += ["-isystem", p]
    import sysconfig
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = ["g++", "-O2", "-std=c++17", "-fPIC", "-w", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
              "-DTORCH_API_INCLUDE_EXTENSION_H", "-I", ext_dir] + inc

    def compile_one(src):
        obj = os.path.join(obj_dir, os.path.basename(src) + ".o")
        cmd = common + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("compile failed: %s\n%s" % (" ".join(cmd), r.stderr[-4000:]))
        return obj

    lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    all_srcs = sorted({x for ss in stale.values() for x in ss})
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        obj_of = dict(zip(all_srcs, ex.map(compile_one, all_srcs)))
    for so, ss in stale.items():
        link = ["g++", "-shared", "-o", so] + [obj_of[x] for x in ss] + [
            "-L", lib_dir, "-Wl,-rpath," + lib_dir, "-ltorch", "-ltorch_cpu", "-lc10"]
        r = subprocess.run(link, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stderr[-4000:])
        if verbose:
            print("built", so)
    return OUT_SO


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    out = build(a.reference, a.force)
    if out is None:
        print("reference checkout not found; nothing built")
        sys.exit(1)
