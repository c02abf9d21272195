"""Build the UNMODIFIED reference CUDA extensions into oracle/_ref/ (test infrastructure only).

The reference (zirui-ray-liu/Exact) ships its pack/unpack, mask and SpMM arithmetic only as CUDA
kernels (exact/exact/cpp_extension/quantization_cuda_kernel.cu, spmm_cuda.cu).  This script
compiles those sources *where they lie* in a checkout of the reference, for sm_100a, against the
installed torch, and leaves two importable torch extensions in oracle/_ref/:

    ref_quantization  <- quantization.cc + quantization_cuda_kernel.cu   (setup.py:14-18)
    ref_spmm          <- spmm.cc + spmm_cuda.cu                          (setup.py:19-21)

Nothing is copied from the reference.  Two headers the 2021-era source includes no longer exist in
torch >= 2.0 (ATen/CUDAGeneratorImpl.h, THC/THCGeneral.h); a compatibility include directory with
one-line forwarding headers is generated next to the build output so the sources compile as they are.

The built modules are used ONLY by tests (to pin the CPU oracle against the reference's own kernels
on a GPU) and by tests/golden/make_ref_vectors.py.  The product never imports them.

usage: python oracle/build_ref.py [--reference /path/to/Exact]
"""
import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def _write_shims(shim_dir):
    os.makedirs(os.path.join(shim_dir, "ATen"), exist_ok=True)
    os.makedirs(os.path.join(shim_dir, "THC"), exist_ok=True)
    with open(os.path.join(shim_dir, "ATen", "CUDAGeneratorImpl.h"), "w") as f:
        f.write("#pragma once\n#include <ATen/cuda/CUDAGeneratorImpl.h>\n#include <ATen/cuda/CUDAContext.h>\n")
    with open(os.path.join(shim_dir, "THC", "THCGeneral.h"), "w") as f:
        f.write("#pragma once\n")
    thc_atomics = os.path.join(shim_dir, "THC", "THCAtomics.cuh")
    with open(thc_atomics, "w") as f:
        f.write("#pragma once\n#include <ATen/cuda/Atomic.cuh>\n")


def build(reference="/root/reference", verbose=False):
    ext_dir = os.path.join(reference, "exact", "exact", "cpp_extension")
    if not os.path.isdir(ext_dir):
        raise FileNotFoundError(f"reference checkout not found at {reference}")
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils import cpp_extension

    shim = os.path.join(OUT, "shim")
    _write_shims(shim)
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "--expt-extended-lambda", "-lineinfo"]
    mods = {
        "ref_quantization": ["quantization.cc", "quantization_cuda_kernel.cu"],
        "ref_spmm": ["spmm.cc", "spmm_cuda.cu"],
    }
    for name, srcs in mods.items():
        bdir = os.path.join(OUT, "build_" + name)
        os.makedirs(bdir, exist_ok=True)
        cpp_extension.load(
            name=name,
            sources=[os.path.join(ext_dir, s) for s in srcs],
            extra_include_paths=[shim, ext_dir],
            extra_cuda_cflags=flags,
            build_directory=bdir,
            verbose=verbose,
            is_python_module=True,
        )
        # keep only the shared object next to the others so that it travels without the ninja tree
        so = os.path.join(bdir, name + ".so")
        dst = os.path.join(OUT, name + ".so")
        if os.path.exists(so):
            import shutil
            shutil.copy2(so, dst)
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.reference, a.verbose))
