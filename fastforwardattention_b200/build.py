"""In-tree build of the native pieces for sm_100a.

    python -m fastforwardattention_b200.build [--force]

  libffa_b200.so       the CUDA kernels behind the C ABI of include/ffa_c_api.h (nvcc)
  ff_attention*.so     the torch extension exposing FastForwardAttn (g++, links the above)

Replaces the reference's setup.py (sm_80/sm_86) and compile.sh (sm_75/80/86): one target
architecture, sm_100a.  Outputs land beside this file so that they are found by relative path.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CUDA_HOME = os.path.dirname(os.path.dirname(NVCC))
LIB = os.path.join(PKG, "libffa_b200.so")
EXT = os.path.join(PKG, "ff_attention" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))

CUDA_SOURCES = ["ffa_decode_kernels.cu", "ffa_c_api.cu", "ffa_no_alloc.cu", "ffa_peer_gather.cu"]
KERNEL_HEADERS = ["ffa_internal.h", "ffa_device_common.cuh", "ffa_stream_kernel.cuh", "ffa_prune_kernels.cuh",
                  "ffa_prune_stream_kernel.cuh"]
CUDA_DEPS = CUDA_SOURCES + KERNEL_HEADERS + [os.path.join(ROOT, "include", "ffa_c_api.h")]
NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d if os.path.isabs(d) else os.path.join(CSRC, d)) > t for d in deps)


def _run(cmd) -> None:
    print("+", " ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def build_library(force: bool = False, verbose_ptxas: bool = False) -> str:
    if force or _stale(LIB, CUDA_DEPS):
        objs = []
        for src in CUDA_SOURCES:
            obj = os.path.join(PKG, "build", src.replace(".cu", ".o"))
            os.makedirs(os.path.dirname(obj), exist_ok=True)
            if force or _stale(obj, CUDA_DEPS if src != "ffa_decode_kernels.cu" else
                               ["ffa_decode_kernels.cu"] + KERNEL_HEADERS):
                _run([NVCC, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose_ptxas else []), "-c",
                      os.path.join(CSRC, src), "-o", obj])
            objs.append(obj)
        _run([NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs])
    return LIB


def build_extension(force: bool = False) -> str:
    src = os.path.join(CSRC, "torch_binding.cpp")
    if force or _stale(EXT, [src, os.path.join(ROOT, "include", "ffa_c_api.h"), LIB]):
        import torch
        from torch.utils.cpp_extension import include_paths

        tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
        inc = [f"-I{p}" for p in include_paths()] + [f"-I{sysconfig.get_paths()['include']}",
                                                     f"-I{CUDA_HOME}/include", f"-I{os.path.join(ROOT, 'include')}"]
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=ff_attention",
              "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
              *inc, src, "-o", EXT, f"-L{PKG}", "-lffa_b200", f"-L{tlib}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
              "-ltorch_cuda", "-ltorch", "-ltorch_python", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}"])
    return EXT


def build_all(force: bool = False) -> None:
    build_library(force)
    build_extension(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
