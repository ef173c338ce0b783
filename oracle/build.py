"""Build recipe of the C oracle: ``python oracle/build.py`` -> oracle/liboracle.so.

Test infrastructure only.  The reference tree itself cannot be compiled for this path (it needs
hipcc/ROCm, MIOpen and the PIM SDK), so there is no oracle/_ref build; the arithmetic of the path
lives in libtorch, which oracle/torch_oracle.py calls directly.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "oracle.c")
LIB = os.path.join(HERE, "liboracle.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    # no -march=native: the library must run on whatever host CPU the GPU box has
    cmd = ["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", "-o", LIB, SRC, "-lm"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("gcc failed:\n" + res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
