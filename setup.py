"""Builds the sm_100a kernel library in-tree:  python setup.py build_ext --inplace

Produces optimus_lm_b200/_C.*.so (PyTorch extension: bindings + all kernels) and
optimus_lm_b200/libolb.so (the same kernels behind a plain C ABI, no Python or torch
dependency).  nvcc cross-compiles for sm_100a, so no GPU is needed to build.
"""
import glob
import os
import subprocess
import sys

from setuptools import setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join("optimus_lm_b200", "csrc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"]

if os.environ.get("OLB_DEBUG_CHECKS", "0") == "1":
    # index checks that record ST_BAD_ARG instead of faulting (csrc/ptx.cuh: OLB_INDEX_OK)
    NVCC_FLAGS.append("-DOLB_DEBUG_CHECKS")

cu_sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
cpp_sources = sorted(glob.glob(os.path.join(CSRC, "*.cpp")))


def build_c_library():
    """libolb.so: every .cu behind the extern "C" API of olb_api.h."""
    out = os.path.join(ROOT, "optimus_lm_b200", "libolb.so")
    srcs = [os.path.join(ROOT, s) for s in cu_sources]
    if os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(s) for s in srcs + glob.glob(
            os.path.join(ROOT, CSRC, "*.h")) + glob.glob(os.path.join(ROOT, CSRC, "*.cuh"))):
        return
    cmd = ["nvcc", "-shared", "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-o", out] + srcs + ["-lcudart"]
    if os.environ.get("OLB_DEBUG_CHECKS", "0") == "1":
        cmd.insert(1, "-DOLB_DEBUG_CHECKS")
    print(" ".join(cmd))
    subprocess.check_call(cmd)


if "build_ext" in sys.argv and os.environ.get("OLB_SKIP_CLIB", "0") != "1":
    build_c_library()

setup(
    name="optimus_lm_b200",
    version="0.1.0",
    packages=[],
    ext_modules=[
        CUDAExtension(
            name="optimus_lm_b200._C",
            sources=cpp_sources + cu_sources,
            include_dirs=[os.path.join(ROOT, CSRC)],
            extra_compile_args={"cxx": ["-O2", "-std=c++17"], "nvcc": NVCC_FLAGS},
        )
    ],
    cmdclass={"build_ext": BuildExtension.with_options(use_ninja=True)},
)
