"""ctypes binding of libplx_sm100.so (the C ABI declared in include/plx_abi.h).

There is no fallback: if the library is missing or a call fails, an exception
is raised.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

from ._paths import LIB_PATH

PLX_BF16, PLX_FP16 = 0, 1
PLX_ERR_UNSUPPORTED = -2
PLX_ERR_STATIC_SCRATCH = -6
DECODE_STATIC_SCRATCH_BYTES = 4 << 20
ABI_VERSION = 2

# every symbol include/plx_abi.h declares
SYMBOLS = (
    "plx_abi_version", "plx_strerror", "plx_kernel_launch_count", "plx_device_error", "plx_device_error_peek",
    "plx_train_workspace_bytes", "plx_train_fwd", "plx_train_bwd", "plx_train_bwd_stages",
    "plx_decode_choose_splits", "plx_decode_choose_splits_gqa", "plx_decode_workspace_bytes", "plx_decode", "plx_decode_static", "plx_decode_partial",
    "plx_decode_merge", "plx_decode_exchange_bytes", "plx_decode_exchange_merge", "plx_decode_partial_exchange",
)
EXCHANGE_MAX_RANKS = 16


class TrainProblem(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("batch", C.c_int32), ("heads_q", C.c_int32), ("heads_kv", C.c_int32),
        ("len_q", C.c_int32), ("len_k", C.c_int32), ("head_dim", C.c_int32), ("window_left", C.c_int32),
        ("qk_scale", C.c_float), ("n_seqs", C.c_int32),
        ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64), ("q_stride_t", C.c_int64),
        ("kv_stride_b", C.c_int64), ("kv_stride_h", C.c_int64), ("kv_stride_t", C.c_int64),
        ("st_stride_b", C.c_int64), ("st_stride_h", C.c_int64), ("st_stride_t", C.c_int64),
        ("cu_seqlens", C.c_void_p),
    ]


class DecodeProblem(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("batch", C.c_int32), ("heads_q", C.c_int32), ("heads_kv", C.c_int32),
        ("cache_len", C.c_int32), ("head_dim", C.c_int32), ("window_left", C.c_int32), ("n_splits", C.c_int32),
        ("qk_scale", C.c_float), ("kv_offset", C.c_int32), ("total_len", C.c_int32),
        ("kv_stride_b", C.c_int64), ("kv_stride_t", C.c_int64), ("kv_stride_h", C.c_int64),
        ("page_table", C.c_void_p), ("page_size", C.c_int32), ("pages_per_seq", C.c_int32),
    ]


class Exchange(C.Structure):
    _fields_ = [
        ("world", C.c_int32), ("rank", C.c_int32), ("n_records", C.c_int32), ("head_dim", C.c_int32),
        ("dtype", C.c_int32), ("wait_ms", C.c_uint32), ("status", C.c_void_p),
        ("inbox", C.c_void_p * EXCHANGE_MAX_RANKS),
    ]


class PlxError(RuntimeError):
    """A libplx_sm100 entry point returned a negative status."""

    def __init__(self, status: int, what: str, msg: str):
        super().__init__(f"{what}: {msg} (status {status})")
        self.status = status


_lock = threading.Lock()
_lib = None


def _declare(lib):
    vp, i32, sz = C.c_void_p, C.c_int32, C.c_size_t
    lib.plx_abi_version.restype = C.c_int
    lib.plx_abi_version.argtypes = []
    lib.plx_strerror.restype = C.c_char_p
    lib.plx_strerror.argtypes = [C.c_int]
    lib.plx_kernel_launch_count.restype = C.c_uint64
    lib.plx_kernel_launch_count.argtypes = []
    lib.plx_device_error.restype = C.c_int
    lib.plx_device_error.argtypes = [C.POINTER(C.c_int32), i32]
    lib.plx_device_error_peek.restype = C.c_int
    lib.plx_device_error_peek.argtypes = [C.POINTER(C.c_int32), i32]
    lib.plx_train_workspace_bytes.restype = C.c_int
    lib.plx_train_workspace_bytes.argtypes = [C.POINTER(TrainProblem), C.POINTER(sz)]
    lib.plx_train_fwd.restype = C.c_int
    lib.plx_train_fwd.argtypes = [C.POINTER(TrainProblem)] + [vp] * 9 + [vp]
    lib.plx_train_bwd.restype = C.c_int
    lib.plx_train_bwd.argtypes = [C.POINTER(TrainProblem)] + [vp] * 14 + [vp, sz, vp]
    lib.plx_train_bwd_stages.restype = C.c_int
    lib.plx_train_bwd_stages.argtypes = [C.POINTER(TrainProblem), i32] + [vp] * 14 + [vp, sz, vp]
    lib.plx_decode_choose_splits.restype = C.c_int
    lib.plx_decode_choose_splits.argtypes = [i32, i32, i32, i32]
    lib.plx_decode_choose_splits_gqa.restype = C.c_int
    lib.plx_decode_choose_splits_gqa.argtypes = [i32, i32, i32, i32, i32]
    lib.plx_decode_workspace_bytes.restype = C.c_int
    lib.plx_decode_workspace_bytes.argtypes = [C.POINTER(DecodeProblem), C.POINTER(sz)]
    lib.plx_decode.restype = C.c_int
    lib.plx_decode.argtypes = [C.POINTER(DecodeProblem)] + [vp] * 7 + [vp, sz, vp]
    lib.plx_decode_static.restype = C.c_int
    lib.plx_decode_static.argtypes = [C.POINTER(DecodeProblem)] + [vp] * 7 + [vp]
    lib.plx_decode_partial.restype = C.c_int
    lib.plx_decode_partial.argtypes = [C.POINTER(DecodeProblem)] + [vp] * 7 + [vp, sz, vp]
    lib.plx_decode_merge.restype = C.c_int
    lib.plx_decode_merge.argtypes = [vp, i32, i32, i32, i32, vp, vp]
    lib.plx_decode_exchange_bytes.restype = sz
    lib.plx_decode_exchange_bytes.argtypes = [i32, i32, i32]
    lib.plx_decode_exchange_merge.restype = C.c_int
    lib.plx_decode_exchange_merge.argtypes = [C.POINTER(Exchange), vp, vp, vp]
    lib.plx_decode_partial_exchange.restype = C.c_int
    lib.plx_decode_partial_exchange.argtypes = [C.POINTER(DecodeProblem), C.POINTER(Exchange)] + [vp] * 7 + [vp, sz, vp]


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"{LIB_PATH} is missing: build it with `python -m parallax_b200.build` "
                        "(needs nvcc; there is no CPU or PyTorch fallback)")
                handle = C.CDLL(LIB_PATH)
                _declare(handle)
                got = handle.plx_abi_version()
                if got != ABI_VERSION:
                    raise RuntimeError(f"libplx_sm100.so has ABI version {got}, expected {ABI_VERSION}")
                _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        raise PlxError(status, what, lib().plx_strerror(status).decode())


def device_error(clear: bool = True) -> int:
    """Error word of the pipelined kernels on the current device (0 = none); synchronises the device."""
    v = C.c_int32(0)
    check(lib().plx_device_error(C.byref(v), 1 if clear else 0), "plx_device_error")
    return int(v.value)


def describe_error(word: int) -> str:
    site = word >> 8
    if 40 <= site < 40 + EXCHANGE_MAX_RANKS:
        return f"the peer-memory exchange gave up waiting for the records of rank {site - 40}"
    return f"a pipelined kernel gave up a bounded wait at site {site}"


def raise_if_device_error(what: str) -> None:
    """Raise :class:`PlxError` if a kernel launched earlier on the current device has reported that it
    gave up a bounded wait (the outputs of that launch are undefined).  Reads the report's copy in
    pinned host memory: no synchronisation, cheap enough to run before every launch; the report is
    acknowledged, so it is raised once.  A report can only be seen once the failing kernel has run,
    i.e. at a later call -- call :func:`device_error` after a synchronisation point to be certain."""
    v = C.c_int32(0)
    check(lib().plx_device_error_peek(C.byref(v), 1), "plx_device_error_peek")
    if v.value != 0:
        raise PlxError(-3, what, f"an earlier launch on this device failed: {describe_error(int(v.value))}; "
                                 "its outputs are undefined")


def launch_count() -> int:
    return int(lib().plx_kernel_launch_count())
