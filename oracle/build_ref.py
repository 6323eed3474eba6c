"""Builds the reference's own operator extension, from its sources where they
lie, into ``oracle/_ref/``.  TEST INFRASTRUCTURE ONLY.

Nothing is copied or patched: the four reference files
(EPPGCN/GCNConv/EPPGCN.cpp, EPPGCN_kernel.cu, cuCompactor.cu and the
cuda_error_check.cu they include) are compiled in place with one
force-included compatibility header (``oracle/torch_compat.h``).  The result
is a Python module named ``eppgcn_reference`` exposing the reference's twelve
operators.  Its CPU operators (build_part, get_ginfo) run anywhere; its CUDA
operators need a GPU and are used by the GPU parity tests as the reference
side.  The reference's own ``setup.py`` passes no architecture flag
(EPPGCN/GCNConv/setup.py:15-16); sm_100 is selected here.

Usage: ``python oracle/build_ref.py [reference_root]``; without an argument the
root is ``$EPPGCN_REFERENCE_ROOT``, else a checkout named ``reference`` beside
this repository.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "eppgcn_reference"
TARGET = os.path.join(OUT, NAME + sysconfig.get_config_var("EXT_SUFFIX"))
DEFAULT_ROOT = os.environ.get("EPPGCN_REFERENCE_ROOT") or os.path.normpath(os.path.join(HERE, "..", "..", "reference"))


def build(reference_root: str = DEFAULT_ROOT, force: bool = False, verbose: bool = True) -> str | None:
    src = os.path.join(reference_root, "EPPGCN", "GCNConv")
    files = [os.path.join(src, f) for f in ("EPPGCN.cpp", "EPPGCN_kernel.cu", "cuCompactor.cu")]
    if not all(os.path.exists(f) for f in files):
        return TARGET if os.path.exists(TARGET) else None
    if os.path.exists(TARGET) and not force:
        return TARGET
    import torch
    from torch.utils.cpp_extension import include_paths
    os.makedirs(OUT, exist_ok=True)
    inc = include_paths("cuda") if "cuda" in include_paths.__code__.co_varnames else include_paths()
    inc += [sysconfig.get_paths()["include"], "/usr/local/cuda/include"]
    common = [f"-DTORCH_EXTENSION_NAME={NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
              f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}",
              "-include", os.path.join(HERE, "torch_compat.h")] + ["-I" + p for p in inc]
    objs = []
    for f in files:
        obj = os.path.join(OUT, os.path.basename(f) + ".o")
        if f.endswith(".cu"):
            cmd = ["nvcc", "-c", f, "-o", obj, "-O3", "-std=c++17", "-w",
                   "-gencode", "arch=compute_100,code=sm_100", "-Xcompiler", "-fPIC",
                   "--expt-relaxed-constexpr", "-D__CUDA_NO_HALF_OPERATORS__",
                   "-D__CUDA_NO_HALF_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__"] + common
        else:
            cmd = ["g++", "-c", f, "-o", obj, "-O3", "-fopenmp", "-std=c++17", "-fPIC", "-w"] + common
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        objs.append(obj)
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    link = ["g++", "-shared", "-o", TARGET, *objs, "-fopenmp", "-L" + torch_lib, "-Wl,-rpath," + torch_lib,
            "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
            "-L/usr/local/cuda/lib64", "-lcudart"]
    if verbose:
        print(" ".join(link), flush=True)
    subprocess.run(link, check=True)
    for o in objs:
        os.remove(o)
    return TARGET


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("--") else DEFAULT_ROOT,
                force="--force" in sys.argv))
