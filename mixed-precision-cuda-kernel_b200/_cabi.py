"""ctypes view of libcherryq.so: one Python function per symbol of include/cherryq.h.

The tests call the C ABI through this module with raw device pointers taken from
torch tensors (`tensor.data_ptr()`); nothing here allocates device memory.
"""
from __future__ import annotations

import ctypes as C
import os

from . import NativeLibraryMissing, lib_path

SYMBOLS = [
    "cq_strerror", "cq_last_cuda_error", "cq_abi_version",
    "cq_layer_init", "cq_layer_prepare", "cq_layer_unprepare", "cq_scratch_bytes", "cq_layer_matvec",
    "cq_vecquant4matmul_cherryq", "cq_vecquant3matmul_cherryq",
    "cq_dequantize3_normal", "cq_dequantize4_normal",
    "cq_cache_clear", "cq_cache_stats", "cq_cache_evict", "cq_poll",
    "cq_pack_tmp_bytes", "cq_pack", "cq_unpack_dense",
    "cq_tlayer_init", "cq_tlayer_prepare", "cq_tlayer_unprepare",
    "cq_layer_matvec_static", "cq_tlayer_gemm_workspace_bytes", "cq_tlayer_gemm",
    "cq_selftest_bounded_wait", "cq_rmsnorm", "cq_rope_cache", "cq_silu_mul", "cq_attn_decode", "cq_attn_decode_workspace_bytes",
    "cq_peer_region_bytes", "cq_peer_region_create", "cq_peer_region_destroy", "cq_peer_region_export",
    "cq_peer_region_open", "cq_peer_region_close", "cq_peer_allgather",
    "cq_rlayer_init", "cq_rlayer_prepare", "cq_rlayer_unprepare", "cq_rlayer_check", "cq_rlayer_matvec", "cq_rlayers_matvec", "cq_rlayer_matvec_host", "cq_rlayer_preferred_rows", "cq_rlayer_matvec_gather", "cq_rlayer_matvec_swiglu",
]


class cq_layer(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("bits", "K", "N", "C", "G", "Kc", "Kp", "Cp", "n_gran", "n_sub", "sets", "gran_bytes", "cher_bytes")]
    _fields_ += [(n, C.c_uint64) for n in ("off_stream", "off_cherry", "off_osh", "off_cidx", "blob_bytes")]
    _fields_ += [("blob", C.c_void_p)]


class cq_tlayer(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("bits", "K", "N", "C", "G", "Kc", "Kp", "Cp", "n_gran", "n_tile", "n_cher", "sets", "gran_bytes",
                 "tile_bytes")]
    _fields_ += [(n, C.c_uint64) for n in ("off_stream", "off_cidx", "off_osh", "blob_bytes")]
    _fields_ += [("blob", C.c_void_p)]


class cq_rlayer(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("bits", "K", "N", "C", "G", "Kc", "NG", "sets", "Cp", "NT", "tile_bytes", "ksplit")]
    _fields_ += [(n, C.c_uint64) for n in ("off_tiles", "off_perm", "off_cidx", "off_work", "blob_bytes")]
    _fields_ += [("blob", C.c_void_p)]


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise NativeLibraryMissing(f"{path} is missing; build it first (there is no CPU fallback)")
    L = C.CDLL(path)
    vp, i32, u64 = C.c_void_p, C.c_int, C.c_uint64
    L.cq_strerror.restype = C.c_char_p
    L.cq_strerror.argtypes = [i32]
    L.cq_scratch_bytes.restype = C.c_size_t
    L.cq_pack_tmp_bytes.restype = C.c_size_t
    L.cq_pack_tmp_bytes.argtypes = [i32]
    L.cq_layer_init.argtypes = [C.POINTER(cq_layer), i32, i32, i32, i32, i32, vp]
    L.cq_layer_prepare.argtypes = [C.POINTER(cq_layer), vp, vp, vp, vp, vp]
    L.cq_layer_unprepare.argtypes = [C.POINTER(cq_layer), vp, vp, vp, vp, vp]
    L.cq_layer_matvec.argtypes = [C.POINTER(cq_layer), vp, i32, vp, i32, i32, i32, vp, vp, vp]
    L.cq_layer_matvec_static.argtypes = [C.POINTER(cq_layer), vp, i32, vp, i32, i32, i32, vp, vp]
    L.cq_rlayer_init.argtypes = [C.POINTER(cq_rlayer), i32, i32, i32, i32, i32, vp]
    L.cq_rlayer_prepare.argtypes = [C.POINTER(cq_rlayer), vp, vp, vp, vp, vp]
    L.cq_rlayer_unprepare.argtypes = [C.POINTER(cq_rlayer), vp, vp, vp, vp, vp]
    L.cq_rlayer_check.argtypes = [C.POINTER(cq_rlayer)]
    L.cq_rlayer_matvec.argtypes = [C.POINTER(cq_rlayer), vp, vp, i32, vp, vp]
    L.cq_rlayer_preferred_rows.argtypes = [C.POINTER(cq_rlayer)]
    L.cq_rlayer_matvec_swiglu.argtypes = [C.POINTER(cq_rlayer), vp, vp, i32, vp, i32, i32, vp, vp]
    L.cq_rlayer_matvec_gather.argtypes = [C.POINTER(cq_rlayer), vp, i32, vp, i32, C.POINTER(vp), i32, i32, C.c_size_t, vp, i32, vp, vp]
    L.cq_rlayer_matvec_host.argtypes = [C.POINTER(cq_rlayer), vp, vp, vp, vp, vp, vp]
    L.cq_rlayers_matvec.argtypes = [C.POINTER(C.POINTER(cq_rlayer)), i32, vp, i32, C.POINTER(vp), i32, i32, i32, vp, vp]
    L.cq_tlayer_init.argtypes = [C.POINTER(cq_tlayer), i32, i32, i32, i32, i32, vp]
    L.cq_tlayer_prepare.argtypes = [C.POINTER(cq_tlayer), vp, vp, vp, vp, vp]
    L.cq_tlayer_unprepare.argtypes = [C.POINTER(cq_tlayer), vp, vp, vp, vp, vp]
    L.cq_tlayer_gemm.argtypes = [C.POINTER(cq_tlayer), vp, i32, vp, i32, i32, i32, vp, vp, vp]
    L.cq_tlayer_gemm_workspace_bytes.argtypes = [C.POINTER(cq_tlayer), i32]
    L.cq_tlayer_gemm_workspace_bytes.restype = C.c_size_t
    L.cq_vecquant4matmul_cherryq.argtypes = [vp] * 6 + [i32] * 6 + [u64, vp]
    L.cq_vecquant3matmul_cherryq.argtypes = [vp] * 6 + [i32] * 7 + [u64, vp]
    L.cq_dequantize3_normal.argtypes = [vp, vp, vp] + [i32] * 5 + [vp]
    L.cq_dequantize4_normal.argtypes = [vp, vp, vp] + [i32] * 5 + [vp]
    L.cq_cache_stats.argtypes = [C.POINTER(C.c_int), C.POINTER(C.c_uint64)]
    L.cq_cache_evict.argtypes = [vp, vp, vp, vp]
    L.cq_poll.argtypes = [vp]
    L.cq_pack.argtypes = [vp, i32, vp] + [i32] * 5 + [vp] * 6
    L.cq_unpack_dense.argtypes = [vp] * 4 + [i32] * 5 + [vp, vp]
    L.cq_peer_region_bytes.argtypes = [C.c_size_t]
    L.cq_peer_region_bytes.restype = C.c_size_t
    L.cq_peer_region_create.argtypes = [C.c_size_t, C.POINTER(C.c_void_p)]
    L.cq_peer_region_destroy.argtypes = [vp]
    L.cq_peer_region_export.argtypes = [vp, C.c_char_p]
    L.cq_peer_region_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    L.cq_peer_region_close.argtypes = [vp]
    L.cq_peer_allgather.argtypes = [C.POINTER(C.c_void_p), i32, i32, C.c_size_t, vp, vp, i32, i32, i32, vp, vp]
    _lib = L
    return L


def strerror(rc: int) -> str:
    return lib().cq_strerror(rc).decode()


def check(rc: int, what: str = "cherryq"):
    if rc != 0:
        extra = f" (cudaError {lib().cq_last_cuda_error()})" if rc == 6 else ""
        raise RuntimeError(f"{what}: {strerror(rc)}{extra}")


def layer_init(bits, K, N, Cn, G, blob_ptr=None) -> cq_layer:
    L = cq_layer()
    check(lib().cq_layer_init(C.byref(L), bits, K, N, Cn, G, blob_ptr), "cq_layer_init")
    return L


def rlayer_init(bits, K, N, Cn, G, blob_ptr=None) -> cq_rlayer:
    L = cq_rlayer()
    check(lib().cq_rlayer_init(C.byref(L), bits, K, N, Cn, G, blob_ptr), "cq_rlayer_init")
    return L


def tlayer_init(bits, K, N, Cn, G, blob_ptr=None) -> cq_tlayer:
    L = cq_tlayer()
    check(lib().cq_tlayer_init(C.byref(L), bits, K, N, Cn, G, blob_ptr), "cq_tlayer_init")
    return L
