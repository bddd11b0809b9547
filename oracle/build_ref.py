"""Builds the reference project's own CUDA extension, unmodified, from the sources where they lie
(csrc/quant_cuda.cpp and csrc/quant_cuda_kernel.cu of the reference checkout) into oracle/_ref/.

TEST INFRASTRUCTURE: the result is the reference's GPU kernel, used as a second oracle at batch 1
(the reference's kernels race in shared memory for larger batches) and timed beside this library's
kernel in bench.py.  Nothing of the product imports it.  The module is compiled under the name
`quant_cuda_ref` so that it can live next to this repository's own `quant_cuda`.

    python oracle/build_ref.py [path of the reference checkout]

Plain nvcc / g++ on the two files (the reference's setup_cuda.py is not run); needs torch's headers.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")


def out_path() -> str:
    return os.path.join(OUT_DIR, "quant_cuda_ref" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build(ref_root: str, verbose: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce

    srcs = [os.path.join(ref_root, "csrc", "quant_cuda.cpp"), os.path.join(ref_root, "csrc", "quant_cuda_kernel.cu")]
    for s in srcs:
        if not os.path.exists(s):
            raise FileNotFoundError(s)
    os.makedirs(OUT_DIR, exist_ok=True)
    out = out_path()
    if os.path.exists(out) and all(os.path.getmtime(s) <= os.path.getmtime(out) for s in srcs):
        return out
    inc = ce.include_paths() + [sysconfig.get_paths()["include"], "/usr/local/cuda/include"]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    common = ["-DTORCH_EXTENSION_NAME=quant_cuda_ref", "-DTORCH_API_INCLUDE_EXTENSION_H",
              f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"] + [f"-I{p}" for p in inc]
    obj_cpp, obj_cu = os.path.join(OUT_DIR, "quant_cuda.o"), os.path.join(OUT_DIR, "quant_cuda_kernel.o")
    cmds = [
        ["g++", "-O2", "-std=c++17", "-fPIC", "-c", srcs[0], "-o", obj_cpp] + common,
        ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-Xptxas", "-O3", "--expt-relaxed-constexpr", "-c", srcs[1], "-o", obj_cu] + common,
        ["g++", "-shared", obj_cpp, obj_cu, "-o", out, f"-L{tlib}", "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python",
         "-lc10_cuda", "-ltorch_cuda", "-L/usr/local/cuda/lib64", "-lcudart", f"-Wl,-rpath,{tlib}"],
    ]
    log = []
    for cmd in cmds:
        res = subprocess.run(cmd, capture_output=True, text=True)
        log.append(" ".join(cmd) + "\n" + res.stdout + res.stderr)
        if res.returncode != 0:
            with open(os.path.join(OUT_DIR, "build.log"), "w") as f:
                f.write("\n".join(log))
            raise RuntimeError("building the reference extension failed:\n" + log[-1][-2000:])
    with open(os.path.join(OUT_DIR, "build.log"), "w") as f:
        f.write("\n".join(log))
    for o in (obj_cpp, obj_cu):
        os.remove(o)
    if verbose:
        print(out)
    return out


def load():
    """Imports the built module (None when it has not been built)."""
    import importlib.util
    path = out_path()
    if not os.path.exists(path):
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location("quant_cuda_ref", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def reference_root() -> str:
    """Where the reference project's checkout is looked for: $CHERRYQ_REFERENCE_ROOT, else a directory
    named `reference` beside this repository."""
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return os.environ.get("CHERRYQ_REFERENCE_ROOT") or os.path.join(os.path.dirname(here), "reference")


if __name__ == "__main__":
    build(sys.argv[1] if len(sys.argv) > 1 else reference_root(), verbose=True)
