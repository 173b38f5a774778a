"""Ahead-of-time build of ``visionrl_b200/_C`` for sm_100a.

Every ``.cu`` / ``.cpp`` under ``visionrl_b200/csrc`` is compiled with
``-gencode arch=compute_100a,code=sm_100a`` (the only target) by ninja through
``torch.utils.cpp_extension.load`` and the resulting shared object is copied next to the
package so that it travels with the source tree.  ``python -m visionrl_b200.ops.build``
rebuilds it; ``-v`` adds ``-Xptxas -v`` (registers, spills, shared memory).
"""

from __future__ import annotations

import glob
import os
import shutil
import sys

PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PKG_DIR, "csrc")
BUILD_DIR = os.path.join(PKG_DIR, "csrc", "build")


def sources() -> list[str]:
    found = sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))
    return found


def build_extension(verbose: bool = False, ptxas_verbose: bool = False) -> str:
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load

    os.makedirs(BUILD_DIR, exist_ok=True)
    cuda_flags = [
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "--use_fast_math", "--expt-relaxed-constexpr", "-U__CUDA_NO_HALF_OPERATORS__",
        "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
        "-U__CUDA_NO_HALF2_OPERATORS__",
    ]
    if ptxas_verbose:
        cuda_flags += ["-Xptxas", "-v"]
    module = load(
        name="_C", sources=sources(), extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=cuda_flags, extra_include_paths=[CSRC],
        extra_ldflags=["-lcuda"], build_directory=BUILD_DIR, verbose=verbose,
        is_python_module=True,
    )
    built = module.__file__
    target = os.path.join(PKG_DIR, os.path.basename(built))
    if os.path.abspath(built) != os.path.abspath(target):
        shutil.copy2(built, target)
    return target


if __name__ == "__main__":
    path = build_extension(verbose=True, ptxas_verbose="-v" in sys.argv)
    print(path)
