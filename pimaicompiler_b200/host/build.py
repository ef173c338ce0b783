"""In-tree build of the C++ host-side mirror (`_pimb200_host`), against this interpreter's libtorch and
libpimb200.so.  Usage: ``python -m pimaicompiler_b200.host.build``."""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
OUT = os.path.join(PKG, "_pimb200_host.so")
SOURCES = ["tensor_ops.cpp", "stream_executor.cpp", "op_executors.cpp", "bindings.cpp"]


def needs_build() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cpp", ".h"))]
    deps.append(os.path.join(ROOT, "include", "pimb200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False) -> str:
    if not force and not needs_build():
        return OUT
    import torch
    from torch.utils import cpp_extension as ce
    from pimaicompiler_b200 import build as libbuild
    libbuild.build()
    inc = [*ce.include_paths(), sysconfig.get_paths()["include"], "/usr/local/cuda/include",
           os.path.join(ROOT, "include"), HERE]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    flags = ["-O2", "-std=c++17", "-fPIC", "-w", "-DTORCH_EXTENSION_NAME=_pimb200_host",
             f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)

    def cc(src: str) -> str:
        obj = os.path.join(objdir, src.replace(".cpp", ".o"))
        cmd = ["g++", *flags, *[f"-I{i}" for i in inc], "-c", os.path.join(HERE, src), "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"g++ failed on {src}:\n{res.stdout}{res.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=4) as ex:
        objs = list(ex.map(cc, SOURCES))
    link = ["g++", "-shared", "-o", OUT, *objs, f"-L{tlib}", "-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda",
            "-ltorch_python", f"-L{PKG}", "-lpimb200", f"-Wl,-rpath,{tlib}", "-Wl,-rpath,$ORIGIN"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
