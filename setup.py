"""Builds the sm_100a extension in-tree: `python setup.py build_ext --inplace`
produces fastcache_b200/_C*.so.  The arch flags are passed explicitly
(-gencode arch=compute_100a,code=sm_100a), which bypasses torch's own arch list;
nvcc cross-compiles without a GPU."""
import glob
import os

from setuptools import setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

ROOT = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join("fastcache_b200", "csrc")
sources = sorted(glob.glob(os.path.join(SRC, "*.cu")) + glob.glob(os.path.join(SRC, "*.cpp")))

nvcc_flags = ["-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"] if os.environ.get("FC_PTXAS_V") else \
             ["-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "--expt-relaxed-constexpr"]

setup(
    name="fastcache_b200",
    version="0.1.0",
    packages=[],
    ext_modules=[CUDAExtension(
        name="fastcache_b200._C",
        sources=sources,
        include_dirs=[os.path.join(ROOT, SRC)],
        extra_compile_args={"cxx": ["-O3", "-std=c++17"], "nvcc": nvcc_flags},
    )],
    cmdclass={"build_ext": BuildExtension.with_options(use_ninja=True)},
)
