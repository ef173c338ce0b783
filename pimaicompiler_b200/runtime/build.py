"""Builds the reference's TorchScript importer, IR and graph passes where they lie (nothing of them is copied into this
repository) and links them with this library's runtime into the pybind module `NNCompiler`.

    python -m pimaicompiler_b200.runtime.build --reference /path/to/PimAiCompiler [--force]

What is compiled from the reference tree, unchanged: ir/source/**/*.cpp and compiler/source/**/*.cpp, except the two
units that no longer compile against libtorch 2.x (importer/utils/attr_parser.cpp, importer/utils/utils.cpp), which
are replaced by compat/*.cpp of this directory.  shim/ supplies <glog/logging.h> and "half.hpp" (absent third-party
headers).  The reference's own runtime (HIP / MIOpen / PIM bound) is not compiled: source/*.cpp of this directory is
the runtime, written against the reference's IR headers, over libpimb200.so.

Outputs go to baseline/_ref/ (git-ignored: they contain compiled reference code): object files under obj/ and
NNCompiler.<abi>.so, which `import NNCompiler` finds once that directory is on sys.path.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
OUT_DIR = os.path.join(ROOT, "baseline", "_ref")
REPLACED = ("frontend/importer/utils/attr_parser.cpp", "frontend/importer/utils/utils.cpp")


def module_path() -> str:
    return os.path.join(OUT_DIR, "NNCompiler" + sysconfig.get_config_var("EXT_SUFFIX"))


def available() -> bool:
    """True when a built module exists (a GPU box uses the prebuilt file; it has no reference tree)."""
    return os.path.exists(module_path())


def _walk_cpp(top: str) -> list[str]:
    out = []
    for d, _, files in os.walk(top):
        out += [os.path.join(d, f) for f in sorted(files) if f.endswith(".cpp")]
    return sorted(out)


def build(reference: str, force: bool = False, jobs: int | None = None) -> str:
    import torch
    from torch.utils import cpp_extension as ce
    from pimaicompiler_b200 import build as libbuild
    libbuild.build()
    if not os.path.isdir(os.path.join(reference, "ir", "include")):
        raise RuntimeError(f"{reference} does not look like the reference tree (no ir/include)")
    obj_dir = os.path.join(OUT_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    ref_src = [f for f in _walk_cpp(os.path.join(reference, "ir", "source")) + _walk_cpp(os.path.join(reference, "compiler", "source"))
               if not f.endswith(REPLACED)]
    own_src = _walk_cpp(os.path.join(HERE, "compat")) + _walk_cpp(os.path.join(HERE, "source")) + \
        [os.path.join(PKG, "host", "tensor_ops.cpp")]
    own_hdr_time = max(os.path.getmtime(os.path.join(d, f)) for top in (os.path.join(HERE, "include"), os.path.join(HERE, "shim"),
                                                                       os.path.join(PKG, "host"), os.path.join(ROOT, "include"))
                       for d, _, fs in os.walk(top) for f in fs if f.endswith((".h", ".hpp")))
    inc = [os.path.join(HERE, "shim"), os.path.join(HERE, "include"), os.path.join(PKG, "host"), os.path.join(ROOT, "include"),
           reference, os.path.join(reference, "ir", "include"), os.path.join(reference, "compiler", "include"),
           *ce.include_paths(), sysconfig.get_paths()["include"], "/usr/local/cuda/include"]
    flags = ["-std=c++17", "-fPIC", "-O1", "-w", "-DTORCH_EXTENSION_NAME=NNCompiler", "-DTORCH_API_INCLUDE_EXTENSION_H",
             f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]

    def cc(src: str) -> str:
        own = not src.startswith(reference)
        tag = os.path.relpath(src, ROOT if own else reference).replace(os.sep, "_")[:-4]
        obj = os.path.join(obj_dir, ("own_" if own else "ref_") + tag + ".o")
        newest = max(os.path.getmtime(src), own_hdr_time if own else 0.0)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > newest:
            return obj
        res = subprocess.run(["g++", *flags, *[f"-I{i}" for i in inc], "-c", src, "-o", obj], capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"g++ failed on {src}:\n{res.stdout}{res.stderr[-4000:]}")
        return obj

    with ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(cc, ref_src + own_src))
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    out = module_path()
    link = ["g++", "-shared", "-o", out, *objs, f"-L{tlib}", "-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda", "-ltorch_cuda",
            "-ltorch_python", f"-L{PKG}", "-lpimb200", "-L/usr/local/cuda/lib64", "-lcudart", f"-Wl,-rpath,{tlib}",
            f"-Wl,-rpath,{PKG}", "-Wl,-rpath,$ORIGIN/../../pimaicompiler_b200"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stdout + res.stderr[-4000:])
    return out


def load():
    """Imports the built module (raises when it was never built)."""
    if not available():
        raise RuntimeError("the NNCompiler module has not been built: python -m pimaicompiler_b200.runtime.build --reference <tree>")
    if OUT_DIR not in sys.path:
        sys.path.insert(0, OUT_DIR)
    import torch  # noqa: F401  (libtorch must be loaded first)
    import NNCompiler
    return NNCompiler


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the PimAiCompiler source tree")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build(a.reference, a.force))
