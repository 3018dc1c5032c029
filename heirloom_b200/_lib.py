"""ctypes loader for libheirloom_b200.so.  There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int64, c_longlong, c_size_t, c_uint64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libheirloom_b200.so"


class HeirloomError(RuntimeError):
    """Raised with the library's message (the C ABI's hl_last_error)."""


class DeviceInfo(Structure):
    _fields_ = [("sm_major", c_int), ("sm_minor", c_int), ("sm_count", c_int), ("total_bytes", c_size_t),
                ("free_bytes", c_size_t), ("supports_tcgen05", c_int)]


class Counters(Structure):
    _fields_ = [(n, c_uint64) for n in ("launches", "gemm_tcgen05_launches", "attention_launches", "h2d_bytes",
                                        "d2h_bytes", "allocations", "allocated_bytes", "nccl_calls", "nccl_bytes",
                                        "gemm_pair_launches")]


class Profile(Structure):
    _fields_ = [("ms", ctypes.c_double * 9), ("work", ctypes.c_double * 9), ("scopes", c_uint64 * 9)]


class AdamWParams(Structure):
    _fields_ = [(n, c_float) for n in ("lr", "beta1", "beta2", "eps", "weight_decay", "clip_scale",
                                       "bias_correction1", "bias_correction2")]


class AdamWTensor(Structure):
    _fields_ = [("param", c_void_p), ("grad", c_void_p), ("m", c_void_p), ("v", c_void_p),
                ("shadow_bf16", c_void_p), ("n", c_uint64)]


class MatrixLayout(Structure):
    _fields_ = [(n, c_longlong) for n in ("rows", "cols", "row_stride", "col_stride", "offset")]


class GemmDesc(Structure):
    _fields_ = [("m", c_int), ("n", c_int), ("k", c_int), ("a_layout", c_int), ("b_layout", c_int),
                ("lda", c_longlong), ("ldb", c_longlong), ("ldc", c_longlong), ("epilogue", c_int),
                ("out_dtype", c_int), ("split_k", c_int), ("ld_aux_in", c_longlong), ("ld_aux_out", c_longlong),
                ("a_k_period", c_int), ("b_k_period", c_int)]


_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise HeirloomError(
                f"{LIB_PATH} is missing: build it with `python -m heirloom_b200.build` (there is no CPU fallback)")
        _lib = ctypes.CDLL(str(LIB_PATH))
        _lib.hl_last_error.restype = c_char_p
        _lib.hl_ctx_stream.restype = c_void_p
        _lib.hl_ctx_stream.argtypes = [c_void_p]
        _lib.hl_buffer_ptr.restype = c_void_p
        _lib.hl_buffer_ptr.argtypes = [c_void_p]
        _lib.hl_buffer_bytes.restype = c_size_t
        _lib.hl_buffer_bytes.argtypes = [c_void_p]
        _lib.hl_adamw_plan_destroy.restype = None
        _lib.hl_adamw_plan_destroy.argtypes = [c_void_p]
        _lib.hl_ctx_destroy.restype = None
        _lib.hl_ctx_destroy.argtypes = [c_void_p]
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise HeirloomError(load().hl_last_error().decode("utf-8", "replace") + f" (code {rc})")
