"""In-tree build of the native parts (no GPU needed: nvcc cross-compiles sm_100a).

  libcherryq.so   the C-ABI library (include/cherryq.h): all CUDA kernels
  quant_cuda*.so  thin PyTorch C++ extension with the reference's module name and
                  signatures (csrc/quant_cuda.cpp:72-77 of the reference project)

Both land next to this file so that they travel with the source tree.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
ROOT = os.path.dirname(HERE)

LIB = os.path.join(HERE, "libcherryq.so")
CUDA_SOURCES = ["cq_api.cu", "cq_layout.cu", "cq_matvec.cu", "cq_rowvec.cu", "cq_pack.cu", "cq_legacy_f32.cu",
                "cq_tile_layout.cu", "cq_prefill.cu", "cq_model_ops.cu", "cq_peer.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--fmad=true",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libcherryq.so")
    return exe


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def cuda_sources():
    return [os.path.join(CSRC, s) for s in CUDA_SOURCES]


def build_lib(force: bool = False, verbose: bool = False) -> str:
    srcs = cuda_sources()
    deps = srcs + [os.path.join(CSRC, "cq_common.cuh"), os.path.join(CSRC, "cq_tile.cuh"),
                   os.path.join(ROOT, "include", "cherryq.h")]
    if not force and _newer(LIB, deps):
        return LIB
    cmd = [_nvcc()] + NVCC_FLAGS + ["-o", LIB] + srcs + ["-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = res.stdout + res.stderr
    with open(os.path.join(HERE, "build_libcherryq.log"), "w") as f:
        f.write(" ".join(cmd) + "\n" + log)
    if verbose or res.returncode != 0:
        print(log)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libcherryq.so")
    return LIB


def ext_path() -> str:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(HERE, "quant_cuda" + suffix)


def build_ext(force: bool = False, verbose: bool = False) -> str:
    """The pybind11/torch shim.  Compiled with g++ only: it contains no device code and
    reaches the kernels through the C ABI of libcherryq.so (rpath $ORIGIN)."""
    import torch
    from torch.utils import cpp_extension as ce

    src = os.path.join(CSRC, "quant_cuda_ext.cpp")
    out = ext_path()
    if not force and _newer(out, [src, os.path.join(ROOT, "include", "cherryq.h")]) and os.path.exists(LIB):
        return out
    build_lib(force=False, verbose=verbose)
    inc = ce.include_paths() + [sysconfig.get_paths()["include"], "/usr/local/cuda/include",
                                os.path.join(ROOT, "include")]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-DTORCH_EXTENSION_NAME=quant_cuda",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    cmd += [f"-I{p}" for p in inc]
    cmd += [src, "-o", out, f"-L{HERE}", "-lcherryq", f"-L{tlib}", "-ltorch", "-ltorch_cpu", "-lc10",
            "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
            "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = res.stdout + res.stderr
    with open(os.path.join(HERE, "build_quant_cuda.log"), "w") as f:
        f.write(" ".join(cmd) + "\n" + log)
    if verbose or res.returncode != 0:
        print(log)
    if res.returncode != 0:
        raise RuntimeError("g++ failed building the quant_cuda extension")
    return out


def build_all(force: bool = False, verbose: bool = False):
    return build_lib(force, verbose), build_ext(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
