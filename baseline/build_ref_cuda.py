"""Builds the reference project's own two CUDA extensions, unmodified, for sm_100a, as the GPU-side baseline.

    python baseline/build_ref_cuda.py /path/to/reference/checkout

The sources are compiled where they lie (nothing is copied into this repository); the two shared objects go to
baseline/_ref/ (git-ignored).  Flags are the reference's own (setup.py:14-27: -O3 -std=c++17 --extended-lambda
--expt-relaxed-constexpr -use_fast_math).  Both extensions register the `quant_ops` dispatcher namespace, as the
product's binding does, so they can only be loaded in a process that has not imported quant_ops_b200:
baseline/time_ref_cuda.py is that process.
"""
from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SOURCES = {
    "ref_cuda_quant_ops": "src/quant_ops/ops/quantization/flatquant/kernels/cuda_quant_kernel.cu",
    "ref_cuda_int4_matmul_ops": "src/quant_ops/ops/quantization/int4_matmul/kernels/cuda_int4_matmul_kernel.cu",
}
NVCC_FLAGS = ["-O3", "-std=c++17", "--extended-lambda", "--expt-relaxed-constexpr", "-use_fast_math",
              "-gencode", "arch=compute_100a,code=sm_100a"]


def main() -> None:
    if len(sys.argv) != 2 or not os.path.isdir(sys.argv[1]):
        raise SystemExit(__doc__)
    ref = os.path.abspath(sys.argv[1])
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils import cpp_extension

    os.makedirs(OUT, exist_ok=True)
    for name, rel in SOURCES.items():
        build_dir = os.path.join(OUT, "build_" + name)
        os.makedirs(build_dir, exist_ok=True)
        cpp_extension.load(name=name, sources=[os.path.join(ref, rel)], extra_cflags=["-O3", "-std=c++17"],
                           extra_cuda_cflags=NVCC_FLAGS, build_directory=build_dir, is_python_module=False, verbose=True)
        built = os.path.join(build_dir, name + ".so")
        os.replace(built, os.path.join(OUT, name + ".so"))
        print("built", os.path.join(OUT, name + ".so"))


if __name__ == "__main__":
    main()
