"""Installer of rosa_soft_b200.

Honours the build switches of the reference's installer (its setup.py:50-96) so that scripts
written for it keep working:

  ROSA_BUILD_EXTENSION=1 (default)   compile the native parts
  USE_CUDA=auto|1 (default auto)     the CUDA variant -- the only one this package has

The reference can also install a pure-PyTorch `reference` variant (ROSA_BUILD_EXTENSION=0) and a
CPU-runtime variant (USE_CUDA=0).  This package is the sm_100a CUDA variant and nothing else: it
has no CPU path to fall back to, so those two settings are refused with an explanation instead of
producing a package that cannot import.  The native parts (librosa_soft_b200.so with the C ABI,
_C.so with the torch operator registration) are built in-tree by rosa_soft_b200/build.py with
nvcc for sm_100a and shipped as package data.
"""
import ast
import importlib.util
import os
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).parent
PACKAGE = "rosa_soft_b200"


def _version() -> str:
    tree = ast.parse((ROOT / PACKAGE / "__init__.py").read_text(encoding="utf-8"))
    for node in tree.body:
        if isinstance(node, ast.Assign) and any(
                isinstance(t, ast.Name) and t.id == "__version__" for t in node.targets):
            return ast.literal_eval(node.value)
    raise RuntimeError("__version__ not found")


def resolve_variant(environ=os.environ) -> str:
    build = environ.get("ROSA_BUILD_EXTENSION", "1").strip().lower()
    if build not in {"0", "1"}:
        raise RuntimeError(f"ROSA_BUILD_EXTENSION must be 0 or 1, got {build!r}")
    cuda = environ.get("USE_CUDA", "auto").strip().lower()
    if cuda not in {"auto", "0", "1"}:
        raise RuntimeError(f"USE_CUDA must be auto, 0, or 1, got {cuda!r}")
    if build == "0" or cuda == "0":
        raise RuntimeError(
            "rosa_soft_b200 only exists as the CUDA variant (sm_100a kernels behind the rosa_soft "
            "operator API); ROSA_BUILD_EXTENSION=0 / USE_CUDA=0 would produce a package without "
            "operators.  Install the reference package for its `reference` or CPU-runtime variant.")
    return "cuda"


class BuildWithNativeParts(build_py):
    def run(self):
        resolve_variant()
        spec = importlib.util.spec_from_file_location("_rosa_build", ROOT / PACKAGE / "build.py")
        builder = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(builder)
        builder.build_all(force=False, verbose=False)
        super().run()


setup(
    name=PACKAGE,
    version=_version(),
    description="sm_100a implementation of the rosa_soft operator family (hard suffix routing "
                "forward, dense surrogate VJP, packed variant, batched hard inference)",
    packages=[PACKAGE],
    package_data={PACKAGE: ["*.so", "csrc/*"]},
    data_files=[("include", ["include/rosa_soft_b200.h"])],
    python_requires=">=3.10",
    install_requires=["torch>=2.11,<2.12"],
    cmdclass={"build_py": BuildWithNativeParts},
    zip_safe=False,
)
