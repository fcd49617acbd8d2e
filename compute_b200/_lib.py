"""ctypes binding of libcudabackend.so (the C ABI declared in include/cudabackend.h).

The library is the product: there is no CPU or PyTorch fallback.  If the shared
object is missing, or no CUDA device is visible when one is needed, calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcudabackend.so")

OK, ERR_INVALID_ARG, ERR_NOT_IMPLEMENTED, ERR_OOM, ERR_CUDA, ERR_TIMEOUT, ERR_NO_DEVICE = range(7)


class BackendError(RuntimeError):
    """An ordinary error returned by the backend (a Go `error` in the reference API)."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


class ErrNotImplemented(BackendError):
    """compute.ErrNotImplemented (compute.go:104-115): callers fall back or skip."""


class QDenseDesc(C.Structure):
    _fields_ = [("M", C.c_int64), ("K", C.c_int64), ("N", C.c_int64),
                ("x_dtype", C.c_int32), ("w_dtype", C.c_int32), ("scale_layout", C.c_int32),
                ("block_size", C.c_int64), ("has_zero_point", C.c_int32), ("has_bias", C.c_int32),
                ("activation", C.c_int32), ("variant", C.c_int32),
                ("gather_ranks", C.c_int32), ("gather_rank", C.c_int32), ("scheme", C.c_int32), ("ggml_type", C.c_int32)]


class QDenseMember(C.Structure):
    _fields_ = [("N", C.c_int64), ("has_bias", C.c_int32), ("activation", C.c_int32)]


class DotDesc(C.Structure):
    _fields_ = [("B", C.c_int64), ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
                ("rhs_transposed", C.c_int32), ("in_dtype", C.c_int32), ("out_dtype", C.c_int32),
                ("variant", C.c_int32), ("has_bias", C.c_int32), ("activation", C.c_int32)]


class SdpaDesc(C.Structure):
    _fields_ = [("B", C.c_int64), ("Hq", C.c_int64), ("Hkv", C.c_int64), ("S", C.c_int64),
                ("Skv", C.c_int64), ("D", C.c_int64), ("layout", C.c_int32), ("dtype", C.c_int32),
                ("scale", C.c_double), ("causal", C.c_int32), ("mask_kind", C.c_int32),
                ("mask_rank", C.c_int32), ("mask_dims", C.c_int64 * 4), ("has_seq_lens", C.c_int32),
                ("bias_rank", C.c_int32), ("bias_dims", C.c_int64 * 4), ("variant", C.c_int32)]


# every symbol include/cudabackend.h declares, with its signature
SIGNATURES = {
    "cb_init": ([C.POINTER(C.c_int)], C.c_int),
    "cb_device_desc": ([C.c_int, C.c_char_p, C.c_size_t], C.c_int),
    "cb_device_sm_count": ([C.c_int, C.POINTER(C.c_int)], C.c_int),
    "cb_last_error": ([], C.c_char_p),
    "cb_status_name": ([C.c_int], C.c_char_p),
    "cb_alloc": ([C.c_int, C.c_size_t, C.POINTER(C.c_void_p)], C.c_int),
    "cb_free": ([C.c_int, C.c_void_p], C.c_int),
    "cb_memset": ([C.c_int, C.c_void_p, C.c_int, C.c_size_t, C.c_void_p], C.c_int),
    "cb_h2d": ([C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p], C.c_int),
    "cb_d2h": ([C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p], C.c_int),
    "cb_d2d": ([C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p], C.c_int),
    "cb_host_alloc": ([C.c_size_t, C.POINTER(C.c_void_p)], C.c_int),
    "cb_host_free": ([C.c_void_p], C.c_int),
    "cb_stream_create": ([C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cb_stream_sync": ([C.c_int, C.c_void_p], C.c_int),
    "cb_stream_destroy": ([C.c_int, C.c_void_p], C.c_int),
    "cb_event_create": ([C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cb_event_record": ([C.c_int, C.c_void_p, C.c_void_p], C.c_int),
    "cb_stream_wait_event": ([C.c_int, C.c_void_p, C.c_void_p], C.c_int),
    "cb_event_elapsed_ms": ([C.c_void_p, C.c_void_p, C.POINTER(C.c_float)], C.c_int),
    "cb_event_destroy": ([C.c_int, C.c_void_p], C.c_int),
    "cb_plan_qdense": ([C.c_int, C.POINTER(QDenseDesc), C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_qdense_group": ([C.c_int, C.POINTER(QDenseDesc), C.POINTER(QDenseMember), C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cb_qdense_decode_static": ([C.c_int, C.POINTER(QDenseDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_void_p, C.c_void_p], C.c_int),
    "cb_plan_dot": ([C.c_int, C.POINTER(DotDesc), C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_sdpa": ([C.c_int, C.POINTER(SdpaDesc), C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_copy": ([C.c_int, C.c_int32, C.c_int64, C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_convert": ([C.c_int, C.c_int32, C.c_int32, C.c_int64, C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_iota": ([C.c_int, C.c_int32, C.c_int32, C.POINTER(C.c_int64), C.c_int32, C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_slice": ([C.c_int, C.c_int32, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int64),
                       C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_transpose": ([C.c_int, C.c_int32, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int32),
                           C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_binary": ([C.c_int, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_unary": ([C.c_int, C.c_int32, C.c_int32, C.c_int64, C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_reduce": ([C.c_int, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int32), C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_broadcast_in_dim": ([C.c_int, C.c_int32, C.c_int32, C.POINTER(C.c_int64), C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int32),
                                  C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_embedding_lookup": ([C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_rms_norm": ([C.c_int, C.c_int32, C.c_int64, C.c_int64, C.c_double, C.c_int32, C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_gelu": ([C.c_int, C.c_int32, C.c_int64, C.c_int32, C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_softmax": ([C.c_int, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_layernorm": ([C.c_int, C.c_int32, C.c_int64, C.c_int64, C.c_double, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_cols_bias": ([C.c_int, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.POINTER(C.c_void_p)], C.c_int),
    "cb_plan_workspace_bytes": ([C.c_void_p, C.POINTER(C.c_size_t)], C.c_int),
    "cb_plan_prepare_workspace": ([C.c_void_p, C.c_void_p, C.c_void_p], C.c_int),
    "cb_plan_kernel_name": ([C.c_void_p], C.c_char_p),
    "cb_plan_grid": ([C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)], C.c_int),
    "cb_launch": ([C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.POINTER(C.c_void_p), C.c_int,
                   C.c_void_p, C.c_void_p], C.c_int),
    "cb_plan_check_status": ([C.c_void_p, C.c_void_p], C.c_int),
    "cb_plan_destroy": ([C.c_void_p], C.c_int),
    "cb_plan_bind": ([C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.POINTER(C.c_void_p), C.c_int, C.c_void_p,
                      C.POINTER(C.c_void_p)], C.c_int),
    "cb_bound_launch": ([C.c_void_p, C.c_void_p], C.c_int),
    "cb_bound_launch_many": ([C.POINTER(C.c_void_p), C.c_int, C.c_void_p], C.c_int),
    "cb_bound_destroy": ([C.c_void_p], C.c_int),
    "cb_ipc_export": ([C.c_int, C.c_void_p, C.c_char_p], C.c_int),
    "cb_ipc_open": ([C.c_int, C.c_char_p, C.POINTER(C.c_void_p)], C.c_int),
    "cb_ipc_close": ([C.c_int, C.c_void_p], C.c_int),
    "cb_peer_signal": ([C.c_int, C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_void_p], C.c_int),
    "cb_peer_wait": ([C.c_int, C.c_void_p, C.c_int, C.c_uint32, C.c_void_p, C.c_void_p], C.c_int),
    "cb_peer_signal_wait": ([C.c_int, C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p], C.c_int),
    "cb_comm_unique_id": ([C.c_char_p], C.c_int),
    "cb_comm_init_rank": ([C.c_int, C.c_int, C.c_int, C.c_char_p, C.POINTER(C.c_void_p)], C.c_int),
    "cb_comm_init_rank_timeout": ([C.c_int, C.c_int, C.c_int, C.c_char_p, C.c_double, C.POINTER(C.c_void_p)], C.c_int),
    "cb_comm_check": ([C.c_void_p], C.c_int),
    "cb_comm_sync": ([C.c_void_p, C.c_void_p, C.c_double], C.c_int),
    "cb_comm_size": ([C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int)], C.c_int),
    "cb_comm_allgather": ([C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p], C.c_int),
    "cb_comm_allreduce": ([C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int32, C.c_int32, C.c_void_p], C.c_int),
    "cb_comm_destroy": ([C.c_void_p], C.c_int),
}

_lib = None


def load() -> C.CDLL:
    """Loads the shared library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m compute_b200.build` "
                "(nvcc, sm_100a). compute_b200 has no CPU or PyTorch fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (args, res) in SIGNATURES.items():
            fn = getattr(lib, name)          # AttributeError if the .so lacks a declared symbol
            fn.argtypes = args
            fn.restype = res
        _lib = lib
    return _lib


def check(status: int) -> None:
    if status == OK:
        return
    lib = load()
    msg = (lib.cb_last_error() or b"").decode() or (lib.cb_status_name(status) or b"").decode()
    if status == ERR_NOT_IMPLEMENTED:
        raise ErrNotImplemented(status, msg)
    raise BackendError(status, msg)
