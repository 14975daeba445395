"""In-tree build of the native parts of rosa_soft_b200 (sm_100a only).

  librosa_soft_b200.so   CUDA kernels + C ABI (include/rosa_soft_b200.h); no torch dependency
  _C.so                  thin torch binding: registers the rosa_soft:: operator schemas and
                         forwards them to the C ABI

Usage: ``python rosa_soft_b200/build.py [--force] [--verbose]`` (run as a script: the package itself refuses to import without its extension).  nvcc cross-compiles without
a GPU; the outputs are git-ignored and travel with the source tree.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "librosa_soft_b200.so")
EXT = os.path.join(PKG, "_C.so")

CUDA_SOURCES = ["plan.cu", "hard_forward.cu", "hard_forward_static.cu", "surrogate_vjp.cu", "vjp_tiled.cu", "vjp_tiled_sweep2.cu", "stream_runtime.cu", "api.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def build_library(force: bool = False, verbose: bool = False) -> str:
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    deps = [os.path.join(CSRC, f) for f in CUDA_SOURCES] + [
        os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "bit_match.cuh"),
        os.path.join(CSRC, "tcgen05.cuh"), os.path.join(CSRC, "vjp_shared.cuh"), os.path.join(CSRC, "vjp_tiled.cuh"), os.path.join(CSRC, "vjp_tiled_sweep2_kernel.inl"),
        os.path.join(ROOT, "include", "rosa_soft_b200.h")]
    if not force and _newer(LIB, deps):
        return LIB
    objdir = os.path.join(PKG, "build")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    procs = []
    for src in CUDA_SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd)))
    for src, p in procs:
        if p.wait() != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    _run([nvcc, "-shared", "-o", LIB, *objs, "-Xcompiler", "-fPIC", "-lcudart_static", "-ldl",
          "-lpthread", "-lrt"], verbose)
    return LIB


def build_extension(force: bool = False, verbose: bool = False) -> str:
    src = os.path.join(CSRC, "torch_binding.cpp")
    deps = [src, os.path.join(ROOT, "include", "rosa_soft_b200.h"), LIB]
    if not force and _newer(EXT, deps):
        return EXT
    import torch
    from torch.utils import cpp_extension

    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-DROSA_WITH_CUDA",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-I" + os.path.join(ROOT, "include")]
    for inc in cpp_extension.include_paths():
        cmd += ["-isystem", inc]
    cmd += ["-isystem", os.path.join(cuda_home, "include"),
            "-isystem", sysconfig.get_paths()["include"]]
    cmd += [src, "-o", EXT, "-L" + PKG, "-l:librosa_soft_b200.so", "-Wl,-rpath,$ORIGIN",
            "-L" + torch_lib, "-Wl,-rpath," + torch_lib,
            "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda"]
    _run(cmd, verbose)
    return EXT


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_library(force, verbose)
    build_extension(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)
    print(EXT)
