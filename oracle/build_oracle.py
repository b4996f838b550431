"""TEST INFRASTRUCTURE ONLY: compile oracle/fgc_oracle.c into oracle/libfgc_oracle.so.

Flags matter for parity: -O2 like the reference, x86-64 baseline (no
-march=native) and -ffp-contract=off so that no fused multiply-add is formed.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "fgc_oracle.c")
OUT = os.path.join(HERE, "libfgc_oracle.so")


def build(force=False, verbose=False):
    if (not force and os.path.exists(OUT)
            and os.path.getmtime(OUT) >= os.path.getmtime(SRC)):
        return OUT
    cmd = ["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off",
           "-fvisibility=hidden", "-Wall", "-o", OUT, SRC, "-lm"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + r.stderr)
    if verbose:
        print("built", OUT)
    return OUT


if __name__ == "__main__":
    build(force=True, verbose=True)
