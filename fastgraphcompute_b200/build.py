"""Build recipe of libfgc_b200.so: nvcc, sm_100a only, in-tree output.

    python fastgraphcompute_b200/build.py [--force] [-v] [--debug]

--debug builds libfgc_b200_debug.so instead: the same sources with -DFGC_DEBUG, i.e. with the
bounds checks of csrc/fgc_common.cuh compiled in (a bad index sets a status bit and the access
is skipped).  Load it with FGC_B200_LIB=<path>.

(run as a script: it must work while the package itself cannot be imported yet)

The shared object has no PyTorch dependency; the Python layer loads it with
ctypes and hands it raw device pointers and the current CUDA stream.
"""
import glob
import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB_PATH = os.path.join(PKG_DIR, "libfgc_b200.so")
DEBUG_LIB_PATH = os.path.join(PKG_DIR, "libfgc_b200_debug.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
    # no --use_fast_math: bin indices and squared distances must round like the CPU reference
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps():
    return sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))


def needs_build(path=LIB_PATH):
    if not os.path.exists(path):
        return True
    t = os.path.getmtime(path)
    return any(os.path.getmtime(p) > t for p in _deps())


def build_library(force=False, verbose=False, extra_flags=(), debug=False):
    """Compile every .cu under csrc/ into one libfgc_b200.so (debug: libfgc_b200_debug.so with
    -DFGC_DEBUG); returns its path."""
    out = DEBUG_LIB_PATH if debug else LIB_PATH
    if not force and not needs_build(out):
        return out
    nvcc = os.environ.get("NVCC", "nvcc")
    flags = list(extra_flags) + (["-DFGC_DEBUG"] if debug else [])
    cmd = [nvcc] + NVCC_FLAGS + flags + ["-I", INCLUDE, "-I", CSRC, "-o", out] + sources()
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n%s\n%s" % (" ".join(cmd), r.stderr[-8000:]))
    if verbose:
        print(r.stderr)
        print("built", out)
    return out


if __name__ == "__main__":
    build_library(force="--force" in sys.argv, verbose=True,
                  extra_flags=["-Xptxas", "-v"] if "-v" in sys.argv else [], debug="--debug" in sys.argv)
