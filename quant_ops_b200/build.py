"""Build recipe for the native parts: the C-ABI library and the thin torch binding.

    python quant_ops_b200/build.py            # both
    python quant_ops_b200/build.py --lib      # libquant_ops_b200.so only (nvcc, seconds)

Everything is built in-tree, for sm_100a only.  No GPU is needed to build.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libquant_ops_b200.so")
CU_SOURCES = ["c_abi.cu", "flatquant_generic.cu", "flatquant_sm100.cu", "flatquant_sm100_n64.cu", "flatquant_sm100_n128.cu", "elementwise.cu", "int4_gemm_generic.cu",
              "int4_gemm_sm100.cu", "int4_gemm_sm100_pair.cu", "int4_gemm_sm100_unpack.cu", "int4_gemm_static.cu", "int4_gemm_skinny.cu", "selftest.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fPIC,-fvisibility=hidden,-O3", "-Xptxas", "-v"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_lib(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(PKG), "include", "quant_ops_b200.h"))
    nvcc = _nvcc()

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ, src.replace(".cu", ".o"))
        path = os.path.join(CSRC, src)
        if force or _stale(obj, [path, __file__] + headers):
            cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("QO_NVCC_EXTRA", "").split(), "-c", path, "-o", obj]
            res = subprocess.run(cmd, capture_output=True, text=True)
            with open(obj + ".log", "w") as fh:
                fh.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
            if res.returncode:
                raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
            if verbose:
                print(res.stderr, file=sys.stderr)
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, len(CU_SOURCES))) as pool:
        objs = list(pool.map(compile_one, CU_SOURCES))
    if force or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-cudart", "static", "-Xlinker", "--no-undefined"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


def build_torch_binding(verbose: bool = False) -> str:
    """Compile csrc/torch_binding.cpp (TORCH_LIBRARY registration over the C ABI) into the package directory."""
    import torch  # noqa: F401
    from torch.utils import cpp_extension

    src = os.path.join(CSRC, "torch_binding.cpp")
    out = os.path.join(PKG, "_torch_binding.so")
    if not _stale(out, [src, LIB, os.path.join(os.path.dirname(PKG), "include", "quant_ops_b200.h")]):
        return out
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    incs = cpp_extension.include_paths() + [os.path.join(os.path.dirname(PKG), "include"),
                                            os.path.join(cuda_home, "include")]
    import sysconfig
    incs.append(sysconfig.get_paths()["include"])
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *[f"-isystem{i}" for i in incs], src, "-o", out,
           f"-L{PKG}", "-l:libquant_ops_b200.so", "-Wl,-rpath,$ORIGIN",
           f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch", f"-Wl,-rpath,{torch_lib}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode:
        raise RuntimeError("g++ failed for torch_binding.cpp:\n" + res.stdout + res.stderr)
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--lib", action="store_true", help="build only the C-ABI library")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    args = ap.parse_args()
    print(build_lib(args.verbose, args.force))
    if not args.lib:
        print(build_torch_binding(args.verbose))


if __name__ == "__main__":
    main()
