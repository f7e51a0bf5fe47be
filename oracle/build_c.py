"""Build recipe of the oracle's C restatement: ``python -m oracle.build_c`` -> ``oracle/libfovi_oracle.so``.
(The reference is pure Python, so there is nothing of it to compile: no ``oracle/_ref`` exists.)"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "fovi_oracle.c")
LIB = os.path.join(HERE, "libfovi_oracle.so")
# AVX2+FMA is present on every x86 host that carries a B200; -march=native would tie the file to the build machine.
FLAGS = ["-O3", "-mavx2", "-mfma", "-ffp-contract=off", "-shared", "-fPIC", "-std=gnu99", "-pthread"]


def build(force=False):
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    r = subprocess.run([os.environ.get("CC", "gcc")] + FLAGS + ["-o", LIB, SRC, "-lm"], capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("gcc failed building libfovi_oracle.so")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
