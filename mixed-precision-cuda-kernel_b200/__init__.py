"""B200 (sm_100a) implementation of the CherryQ quantized-linear hot path.

Layout of the package:
  csrc/            CUDA kernels + the C ABI (include/cherryq.h) + the torch shim
  _build.py        in-tree build (nvcc / g++)
  _cabi.py         ctypes view of libcherryq.so (used by tests and tools)
  quantizer.py     FullSymQuantizer          (reference: llama/quantizer.py)
  cherry_linear.py training-side QuantLinear (reference: llama/cherry_linear.py)
  qlinear.py       packed inference QuantLinear (reference: llama/qlinear.py)
  parallel.py      column-parallel sharding of a quantized linear over GPUs

There is no CPU implementation of the kernels: every op raises if the native
library is missing or no CUDA device is present.
"""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys

__all__ = ["quant_cuda", "load_quant_cuda", "lib_path", "ext_path", "NativeLibraryMissing"]

_HERE = os.path.dirname(os.path.abspath(__file__))


class NativeLibraryMissing(RuntimeError):
    pass


def lib_path() -> str:
    """libcherryq.so next to this file; CHERRYQ_LIB overrides it (to try another build)."""
    return os.environ.get("CHERRYQ_LIB") or os.path.join(_HERE, "libcherryq.so")


def ext_path() -> str:
    import sysconfig
    return os.path.join(_HERE, "quant_cuda" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


_quant_cuda = None


def load_quant_cuda():
    """Imports the compiled `quant_cuda` extension that sits in this directory and
    registers it as the top-level module `quant_cuda`, the name the reference's
    llama/qlinear.py:10 imports."""
    global _quant_cuda
    if _quant_cuda is not None:
        return _quant_cuda
    path = ext_path()
    if not (os.path.exists(path) and os.path.exists(lib_path())):
        raise NativeLibraryMissing(
            f"{path} or {lib_path()} is missing: build them with "
            "`python -c 'import __graft_entry__ as g; g.build()'` (needs nvcc and g++). "
            "There is no CPU fallback.")
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    spec = importlib.util.spec_from_file_location("quant_cuda", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules["quant_cuda"] = mod
    _quant_cuda = mod
    return mod


def __getattr__(name):
    if name == "quant_cuda":
        return load_quant_cuda()
    if name in ("QuantLinear", "PackedQuantLinear"):
        return importlib.import_module(".qlinear", __name__).QuantLinear
    if name in ("CherryLinear", "QuantLinearForTraining"):
        return importlib.import_module(".cherry_linear", __name__).QuantLinear
    if name in ("FullSymQuantizer", "Quantizer"):
        return getattr(importlib.import_module(".quantizer", __name__), name)
    raise AttributeError(name)
