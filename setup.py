"""Build script of the `penny_cpp` extension (sm_100a only).

    python setup.py build_ext --inplace

puts penny_cpp.*.so and libpenny_sim.so at the repository root, next to the
`penny_b200` / `penny` packages.  Unlike the reference's setup.py (which links
NVSHMEM and leaves the GPU architecture to torch's defaults, setup.py:16-32)
this links nothing but the CUDA runtime: the driver API is resolved at run time
through cudaGetDriverEntryPoint, so the module imports on a machine without a
GPU or libcuda.
"""
import os
import subprocess
import sys

import setuptools
import torch
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

ROOT = os.path.dirname(os.path.abspath(__file__))

CUDA_SOURCES = [
    "csrc/all_reduce_oneshot.cu",
    "csrc/all_reduce_twoshot.cu",
    "csrc/all_reduce_ring_simple.cu",
    "csrc/all_reduce_ring_standard.cu",
    "csrc/all_reduce_double_ring.cu",
    "csrc/all_reduce_tree.cu",
    "csrc/all_reduce_nvls.cu",
    "csrc/exchange.cu",
    "csrc/fused_ar_rmsnorm.cu",
    "csrc/custom_all_reduce.cu",
    "csrc/comm.cu",
    "csrc/decode_kernels.cu",
    "csrc/decode_attention_fused.cu",
    "csrc/gemm_sm100.cu",
    "csrc/gemm_fused_sm100.cu",
    "csrc/gemm_decode_sm100.cu",
    "csrc/moe_dispatch_combine.cu",
    "csrc/moe_routing.cu",
]
CPP_SOURCES = [
    "csrc/torch_interface.cpp",
    "csrc/custom_all_reduce_binding.cpp",
    "csrc/gemm_binding.cpp",
    "csrc/decode_binding.cpp",
    "csrc/bootstrap.cpp",
    "csrc/symm_heap.cpp",
]

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "--expt-relaxed-constexpr",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-Wno-sign-compare", "-Wno-unused-variable"]


def build_host_sim(out_dir=ROOT):
    """The host protocol simulator: plain C++, no CUDA, no torch."""
    out = os.path.join(out_dir, "libpenny_sim.so")
    src = os.path.join(ROOT, "csrc", "sim", "host_sim.cpp")
    deps = [src] + [os.path.join(ROOT, "csrc", f) for f in os.listdir(os.path.join(ROOT, "csrc"))
                    if f.endswith((".h", ".cuh"))]
    if os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in deps):
        return out
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-pthread", "-o", out, src]
    subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    build_host_sim()
    setuptools.setup(
        name="penny_b200",
        version="0.1.0",
        packages=setuptools.find_packages(include=["penny_b200", "penny_b200.*", "penny", "penny.*"]),
        ext_modules=[
            CUDAExtension(
                name="penny_cpp",
                sources=CPP_SOURCES + CUDA_SOURCES,
                include_dirs=[os.path.join(ROOT, "csrc")],
                extra_compile_args={"cxx": CXX_FLAGS, "nvcc": NVCC_FLAGS},
                # so that `import penny_cpp` finds libc10 / libtorch even when torch was not imported first
                extra_link_args=["-Wl,-rpath," + os.path.join(os.path.dirname(torch.__file__), "lib")],
            )
        ],
        cmdclass={"build_ext": BuildExtension.with_options(use_ninja=True)},
    )
