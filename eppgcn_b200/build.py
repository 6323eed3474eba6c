"""In-tree build of the native pieces.

``libeppgcn_b200.so``  the C-ABI library (CUDA kernels for sm_100a + host
                       helpers), compiled with nvcc; no torch headers.
``GNNAdvisor*.so``     the torch extension that exposes the reference's
                       operator API on top of the C-ABI library.

Both land next to this file so they travel with the source tree.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_NAME = "libeppgcn_b200.so"
LIB_PATH = os.path.join(HERE, LIB_NAME)
DEBUG_LIB_PATH = os.path.join(HERE, "libeppgcn_b200_debug.so")
PROBE_PATH = os.path.join(HERE, "libeppgcn_probe.so")
EXT_NAME = "GNNAdvisor"
EXT_PATH = os.path.join(HERE, EXT_NAME + sysconfig.get_config_var("EXT_SUFFIX"))

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
LIB_SOURCES = ["spmm.cu", "tiled_spmm.cu", "update.cu", "prep.cu", "exchange.cu", "host.cu"]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build eppgcn_b200")
    return nvcc


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd: list[str], verbose: bool):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr, flush=True)


def build_library(force: bool = False, verbose: bool = False, ptxas_info: bool = False,
                  debug_bounds: bool = False) -> str:
    """``debug_bounds``: the bounds-checking build (``-DEPP_DEBUG_BOUNDS``) as a library of its own,
    ``libeppgcn_b200_debug.so``, which ``capi`` loads when ``EPPGCN_B200_DEBUG_BOUNDS=1`` is set."""
    srcs = [os.path.join(CSRC, s) for s in LIB_SOURCES]
    deps = srcs + [os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "rowio.cuh"),
                   os.path.join(HERE, "..", "include", "eppgcn_b200.h"), __file__]
    target = DEBUG_LIB_PATH if debug_bounds else LIB_PATH
    if force or _stale(target, deps):
        flags = list(NVCC_FLAGS)
        if ptxas_info:
            flags += ["-Xptxas", "-v"]
        if debug_bounds:
            flags += ["-DEPP_DEBUG_BOUNDS"]
        _run([_nvcc(), *flags, "-shared", "-o", target, *srcs], verbose or ptxas_info)
    return target


def build_probe(force: bool = False, verbose: bool = False) -> str:
    """The benchmark's measurement aid (bare gather), a library of its own:
    nothing in the package loads it."""
    src = os.path.join(CSRC, "bench", "gather_probe.cu")
    if force or _stale(PROBE_PATH, [src, os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "rowio.cuh"), __file__]):
        _run([_nvcc(), *NVCC_FLAGS, "-shared", "-o", PROBE_PATH, src], verbose)
    return PROBE_PATH


def build_extension(force: bool = False, verbose: bool = False) -> str:
    """g++ build of the pybind/torch layer; links the C-ABI library by rpath."""
    build_library(force=False, verbose=verbose)
    src = os.path.join(CSRC, "gnnadvisor_ext.cpp")
    deps = [src, os.path.join(HERE, "..", "include", "eppgcn_b200.h"), __file__]
    if not (force or _stale(EXT_PATH, deps)):
        return EXT_PATH
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths
    inc = include_paths("cuda") if "cuda" in include_paths.__code__.co_varnames else include_paths()
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    if os.path.join(cuda_home, "include") not in inc:
        inc.append(os.path.join(cuda_home, "include"))
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           f"-DTORCH_EXTENSION_NAME={EXT_NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}",
           "-I" + sysconfig.get_paths()["include"], *["-I" + p for p in inc],
           "-I" + os.path.join(HERE, "..", "include"),
           src, "-o", EXT_PATH,
           "-L" + HERE, "-leppgcn_b200", "-Wl,-rpath,$ORIGIN",
           "-L" + torch_lib, "-Wl,-rpath," + torch_lib,
           "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
           "-L" + os.path.join(cuda_home, "lib64"), "-lcudart"]
    _run(cmd, verbose)
    return EXT_PATH


def build_all(force: bool = False, verbose: bool = False):
    build_library(force, verbose)
    build_extension(force, verbose)
    build_probe(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    if "--debug-bounds" in sys.argv:
        build_library(force="--force" in sys.argv, verbose=True, debug_bounds=True)
