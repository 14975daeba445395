"""Compile the reference's own RosaRuntime (CPU suffix automaton) into oracle/_ref/.

The single source file is compiled where it lies in the mounted reference tree
(``$ROSA_REFERENCE_ROOT``, or a checkout named ``reference`` beside this repository); nothing is copied into
this repository and the output directory is git-ignored.  The shared object is
used by the tests to validate the oracle's restatement of the match semantics
and by the benchmark as the reference CPU baseline of the hard-inference path.

Usage: python oracle/build_ref.py            (no-op when the reference is absent)
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT_LIB = os.path.join(OUT_DIR, "librosa_runtime_ref.so")


def build(reference_root: str | None = None, force: bool = False) -> str | None:
    root = (reference_root or os.environ.get("ROSA_REFERENCE_ROOT")
            or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
    src = os.path.join(root, "rosa_soft", "csrc", "rosa_runtime.cpp")
    if not os.path.exists(src):
        return OUT_LIB if os.path.exists(OUT_LIB) else None
    if os.path.exists(OUT_LIB) and not force:
        return OUT_LIB
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    os.makedirs(OUT_DIR, exist_ok=True)
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    cmd = [cxx, "-O3", "-std=c++17", "-fPIC", "-shared", "-fopenmp",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    for inc in cpp_extension.include_paths():
        cmd += ["-isystem", inc]
    cmd += ["-isystem", sysconfig.get_paths()["include"]]
    cmd += [src, "-o", OUT_LIB, "-L" + torch_lib, "-Wl,-rpath," + torch_lib,
            "-ltorch", "-ltorch_cpu", "-lc10"]
    subprocess.check_call(cmd)
    return OUT_LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv)
    print(path or "reference source not present; nothing built")
