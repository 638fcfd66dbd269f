"""Build script for bluefog_b200.

`python setup.py build_ext --inplace` compiles the native runtime and every CUDA kernel
for sm_100a into bluefog_b200/_C*.so (in-tree, so that the built library travels with the
source tree).  Role of the reference's setup.py (setup.py:101-602) without its MPI/NCCL
probing: the only dependencies are PyTorch's headers and the CUDA toolkit.
"""
import glob
import os

from setuptools import find_packages, setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join("bluefog_b200", "csrc")


def sources():
    files = [os.path.join(CSRC, "bindings.cc")]
    files += sorted(glob.glob(os.path.join(CSRC, "common", "*.cc")))
    files += sorted(glob.glob(os.path.join(CSRC, "cuda", "*.cc")))
    files += sorted(glob.glob(os.path.join(CSRC, "cuda", "*.cu")))
    return files


NVCC_FLAGS = [
    "-O3", "-std=c++17", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "--expt-relaxed-constexpr", "--use_fast_math", "-Xptxas", "-v",
]

CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-sign-compare", "-Wno-unused-function"]
LINK_FLAGS = ["-Wl,--strip-debug"]
if os.environ.get("BLUEFOG_B200_TSAN") == "1":
    # ThreadSanitizer build of the host runtime (the .cc files; device code is not instrumented).  Build it beside the
    # regular library, not over it, and load it with BLUEFOG_B200_NATIVE (see `make tsan`):
    #   CC=/usr/bin/gcc CXX=/usr/bin/g++ BLUEFOG_B200_TSAN=1 python setup.py build_ext --build-lib build/tsan --build-temp build/tsan_tmp
    CXX_FLAGS = ["-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=thread", "-std=c++17", "-fPIC", "-Wno-sign-compare"]
    LINK_FLAGS = ["-fsanitize=thread"]

ext = CUDAExtension(
    name="bluefog_b200._C",
    sources=sources(),
    include_dirs=[os.path.join(ROOT, CSRC)],
    extra_compile_args={"cxx": CXX_FLAGS, "nvcc": NVCC_FLAGS},
    libraries=["rt"],
    extra_link_args=LINK_FLAGS,
)

setup(
    name="bluefog_b200",
    version="0.1.0",
    description="Blackwell-native decentralized training library with BlueFog's capabilities",
    packages=find_packages(include=["bluefog_b200", "bluefog_b200.*"]),
    ext_modules=[ext],
    cmdclass={"build_ext": BuildExtension.with_options(use_ninja=True)},
    entry_points={"console_scripts": ["bfrun = bluefog_b200.run.run:main", "ibfrun = bluefog_b200.run.interactive_run:main"]},
)
