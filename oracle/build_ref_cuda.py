"""Builds the reference's own hand-written CUDA DSQG extension for sm_100a, from its source where
it lies in the reference checkout, into oracle/_ref/ (git-ignored; built files only, no source is
copied).  Test / measurement infrastructure, never part of the product.

    python oracle/build_ref_cuda.py [/path/to/reference]

Source: kernels/dsqg_cuda/dsqg_cuda_kernel.cu of the DWARF checkout (pybind11 module with
forward/backward, d50 offset set 0..40,128,384,1536, head width 32 or 48), compiled with the flags
the reference's loader uses (kernels/dsqg_cuda/dsqg_cuda.py:20-30) plus the sm_100a target.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def build(reference_root="/root/reference", verbose=False):
    src = os.path.join(reference_root, "kernels", "dsqg_cuda", "dsqg_cuda_kernel.cu")
    if not os.path.exists(src):
        raise FileNotFoundError(src)
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load
    load(name="dsqg_cuda_ref", sources=[src], build_directory=OUT, is_python_module=True, verbose=verbose,
         extra_cuda_cflags=["-O3", "--use_fast_math", "-std=c++17", "-lineinfo",
                            "-gencode", "arch=compute_100a,code=sm_100a"])
    return os.path.join(OUT, "dsqg_cuda_ref.so")


if __name__ == "__main__":
    print(build(*(sys.argv[1:2]), verbose=True))
