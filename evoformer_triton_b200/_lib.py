"""ctypes binding of libevoattn.so (the C ABI declared in include/evoattn.h)."""
from __future__ import annotations

import ctypes as C
import os
import threading

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libevoattn.so")

ABI_VERSION = 3
BF16, FP16, FP32 = 0, 1, 2
MASK_NONE, MASK_BOOL, MASK_ADD_F32, MASK_ADD_SAME = 0, 1, 2, 3
FLAG_FORCE_GENERIC = 1
BIAS_F32, BIAS_SAME = 0, 1
PATH_NONE, PATH_GENERIC, PATH_TCGEN05 = 0, 1, 2

SYMBOLS = (
    "evoattn_abi_version", "evoattn_strerror", "evoattn_fwd", "evoattn_bwd_workspace_bytes",
    "evoattn_bwd", "evoattn_bwd_static_scratch", "evoattn_last_path", "evoattn_last_launch_count",
    "evoattn_peer_data_bytes", "evoattn_peer_flag_bytes", "evoattn_peer_buffer_create", "evoattn_peer_buffer_open",
    "evoattn_peer_buffer_close", "evoattn_peer_buffer_destroy", "evoattn_peer_allreduce_f32",
    "evoattn_bias_to_heads_first", "evoattn_dbias_to_heads_last",
)
STATIC_SCRATCH_BYTES = 64 << 20


class FwdParams(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32),
        ("B", C.c_int32), ("H", C.c_int32), ("S", C.c_int32), ("R", C.c_int32), ("D", C.c_int32),
        ("scale", C.c_float),
        ("flags", C.c_uint32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("lse", C.c_void_p),
        ("q_stride", C.c_int64 * 4), ("k_stride", C.c_int64 * 4),
        ("v_stride", C.c_int64 * 4), ("o_stride", C.c_int64 * 4),
        ("mask", C.c_void_p),
        ("mask_kind", C.c_int32), ("bias_dtype", C.c_int32),
        ("mask_stride", C.c_int64 * 3),
        ("bias", C.c_void_p),
        ("bias_stride", C.c_int64 * 3),
        ("status", C.c_void_p),
        ("gate", C.c_void_p),
        ("gate_stride", C.c_int64 * 4),
    ]


class PeerAllReduceParams(C.Structure):
    _fields_ = [
        ("world", C.c_int32), ("rank", C.c_int32),
        ("bufs", C.POINTER(C.c_void_p)), ("flags", C.POINTER(C.c_void_p)),
        ("count", C.c_uint64), ("epoch", C.c_uint32),
        ("status", C.c_void_p),
    ]


class BwdParams(C.Structure):
    _fields_ = [
        ("fwd", FwdParams),
        ("d_o", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p), ("dbias", C.c_void_p),
        ("do_stride", C.c_int64 * 4), ("dq_stride", C.c_int64 * 4),
        ("dk_stride", C.c_int64 * 4), ("dv_stride", C.c_int64 * 4),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("dgate", C.c_void_p),
        ("dgate_stride", C.c_int64 * 4),
        ("dmask", C.c_void_p),
        ("exchange", C.POINTER(PeerAllReduceParams)),
    ]


_lib = None
_lock = threading.Lock()


def load() -> C.CDLL:
    """Load the shared library; raise if it has not been built (there is no fallback)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m evoformer_triton_b200.build` "
                "(needs nvcc with sm_100a support). There is no CPU or PyTorch fallback.")
        lib = C.CDLL(LIB_PATH)
        lib.evoattn_abi_version.restype = C.c_int
        lib.evoattn_strerror.restype = C.c_char_p
        lib.evoattn_strerror.argtypes = [C.c_int]
        lib.evoattn_fwd.restype = C.c_int
        lib.evoattn_fwd.argtypes = [C.POINTER(FwdParams), C.c_void_p]
        lib.evoattn_bwd_workspace_bytes.restype = C.c_size_t
        lib.evoattn_bwd_workspace_bytes.argtypes = [C.POINTER(BwdParams)]
        lib.evoattn_bwd.restype = C.c_int
        lib.evoattn_bwd.argtypes = [C.POINTER(BwdParams), C.c_void_p]
        lib.evoattn_bwd_static_scratch.restype = C.c_int
        lib.evoattn_bwd_static_scratch.argtypes = [C.POINTER(BwdParams), C.c_void_p]
        lib.evoattn_last_path.restype = C.c_int
        lib.evoattn_last_launch_count.restype = C.c_int
        lib.evoattn_peer_flag_bytes.restype = C.c_size_t
        lib.evoattn_peer_data_bytes.restype = C.c_size_t
        lib.evoattn_peer_data_bytes.argtypes = [C.c_uint64, C.c_int]
        lib.evoattn_peer_buffer_create.restype = C.c_int
        lib.evoattn_peer_buffer_create.argtypes = [C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]
        lib.evoattn_peer_buffer_open.restype = C.c_int
        lib.evoattn_peer_buffer_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
        lib.evoattn_peer_buffer_close.restype = C.c_int
        lib.evoattn_peer_buffer_close.argtypes = [C.c_void_p]
        lib.evoattn_peer_buffer_destroy.restype = C.c_int
        lib.evoattn_peer_buffer_destroy.argtypes = [C.c_void_p]
        for name in ("evoattn_bias_to_heads_first", "evoattn_dbias_to_heads_last"):
            fn = getattr(lib, name)
            fn.restype = C.c_int
            fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        lib.evoattn_peer_allreduce_f32.restype = C.c_int
        lib.evoattn_peer_allreduce_f32.argtypes = [C.POINTER(PeerAllReduceParams), C.c_void_p]
        if lib.evoattn_abi_version() != ABI_VERSION:
            raise RuntimeError("libevoattn.so ABI version mismatch; rebuild it")
        _lib = lib
    return _lib


def strerror(rc: int) -> str:
    return load().evoattn_strerror(rc).decode()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed: {strerror(rc)} (status {rc})")
