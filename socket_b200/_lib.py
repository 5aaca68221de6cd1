"""ctypes binding of the C-ABI library `libsocket_b200.so` (declared in
`include/socket_b200.h`).  There is no fallback: if the library is missing, importing an
operator raises."""
from __future__ import annotations

import ctypes as C
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libsocket_b200.so")

SK_F32, SK_BF16, SK_F16 = 0, 1, 2
DTYPE_CODE = {torch.float32: SK_F32, torch.bfloat16: SK_BF16, torch.float16: SK_F16}

SK_DEV_POS_OUT_OF_RANGE = 1
SK_DEV_INDEX_OUT_OF_RANGE = 2
SK_DEV_WAIT_TIMEOUT = 4
SK_SPARSE_DECODE_STATIC_BYTES = 2 << 20


class SocketError(RuntimeError):
    """An entry point of the CUDA library returned a non-zero status."""


class DecodeParams(C.Structure):
    """Mirror of `sk_decode_params`."""
    _fields_ = [
        ("q", C.c_void_p), ("k_new", C.c_void_p), ("v_new", C.c_void_p), ("input_pos", C.c_void_p),
        ("planes", C.c_void_p), ("protos_T", C.c_void_p), ("temperature", C.c_float),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("codes", C.c_void_p),
        ("v_norm", C.c_void_p), ("prefill_len", C.c_void_p),
        ("out", C.c_void_p), ("list", C.c_void_p), ("list_len", C.c_void_p),
        ("list_row_stride", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
        ("q_dtype", C.c_int), ("kv_dtype", C.c_int), ("plane_dtype", C.c_int),
        ("B", C.c_int), ("H", C.c_int), ("Hkv", C.c_int), ("D", C.c_int), ("L", C.c_int),
        ("P", C.c_int), ("R", C.c_int),
        ("Tcap", C.c_int64), ("T_max", C.c_int64), ("M", C.c_int64),
        ("sink", C.c_int), ("window", C.c_int), ("select_path", C.c_int),
    ]


_i, _i64, _p, _f, _sz = C.c_int, C.c_int64, C.c_void_p, C.c_float, C.c_size_t

# name -> (restype, argtypes); the order follows include/socket_b200.h
SIGNATURES = {
    "sk_abi_version": (_i, []),
    "sk_status_string": (C.c_char_p, [_i]),
    "sk_last_error": (C.c_char_p, []),
    "sk_hash_keys": (_i, [_p, _i, _i64, _p, _i, _i64, _i, _i, _i, _p, _i, _i64, _p]),
    "sk_kv_append": (_i, [_p, _p, _i, _p, _p, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i64, _i, _i, _p]),
    "sk_hash_keys_tc_workspace_bytes": (_sz, [_i64]),
    "sk_hash_keys_tc": (_i, [_p, _i64, _p, _i64, _i, _i, _i, _p, _i64, _p, _p, _sz, _p, _p]),
    "sk_kv_append_tc_workspace_bytes": (_sz, [_i, _i, _i]),
    "sk_kv_append_tc": (_i, [_p, _p, _i, _p, _p, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i64, _i, _i,
                             _p, _sz, _p]),
    "sk_rope_split": (_i, [_p, _i, _p, _i, _p, _i, _i, _i, _i, _i64, _p, _p, _p, _p, _p]),
    "sk_gemv_allreduce_buffer_bytes": (_sz, [_i, _i, _i]),
    "sk_gemv_allreduce": (_i, [_p, _p, _i64, _p, _p, _i, _i, _i, _i, _p, _i, _i, _i, _p, _p, _p]),
    "sk_lut_head_tile": (_i, [_i]),
    "sk_soft_hash": (_i, [_p, _i, _p, _i, _p, _f, _i, _i, _i, _i, _i, _i, _i, _p, _p, _p]),
    "sk_lut_from_probs": (_i, [_p, _i, _i, _i, _i, _i, _i, _p, _p]),
    "sk_score": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i64, _p, _i64, _p, _i64, _p, _p]),
    "sk_score_compat": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i64, _p]),
    "sk_list_len": (_i64, [_i64, _i, _i, _i64]),
    "sk_select_list": (_i, [_p, _i64, _p, _i64, _i64, _p, _i64, _i, _i, _i, _p, _i64, _p, _p, _p]),
    "sk_score_select_applicable": (_i, [_i, _i, _i, _i, _i, _i64, _i64]),
    "sk_score_select_workspace_bytes": (_sz, [_i, _i, _i, _i, _i64, _i64]),
    "sk_score_filter": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i64, _p, _i64, _i64, _p, _sz, _p, _p]),
    "sk_select_candidates": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i64, _p, _i64, _i64, _i, _i, _p, _i64, _p,
                                  _p, _sz, _p, _p]),
    "sk_score_select_list": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i64, _p, _i64, _i64, _i, _i, _p, _i64, _p,
                                  _p, _sz, _p, _p]),
    "sk_packed_table_bytes": (_sz, [_i, _i, _i]),
    "sk_packed_applicable": (_i, [_i, _i, _i, _i, _i, _i64, _i64]),
    "sk_packed_preferred": (_i, [_i, _i, _i, _i, _i, _i64, _i64]),
    "sk_soft_hash_packed": (_i, [_p, _i, _p, _i, _p, _f, _i, _i, _i, _i, _i, _i, _i, _p, _p, _p]),
    "sk_score_select_packed": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i64, _p, _i64, _i64, _i, _i, _p, _i64,
                                    _p, _p, _sz, _p, _i, _p]),
    "sk_score_select_cluster_size": (_i, [_i, _i, _i, _i, _i, _i64, _i64]),
    "sk_score_select_cluster": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i64, _p, _i64, _i64, _i, _i, _p, _i64, _p,
                                     _p, _p]),
    "sk_sparse_decode_workspace_bytes": (_sz, [_i, _i, _i, _i64]),
    "sk_sparse_decode": (_i, [_p, _i, _p, _p, _i, _i64, _i64, _i64, _p, _i64, _p, _i64, _p, _i, _i,
                              _i, _i, _i64, _p, _p, _sz, _p, _p]),
    "sk_sparse_decode_static": (_i, [_p, _i, _p, _p, _i, _i64, _i64, _i64, _p, _i64, _p, _i64, _p, _i, _i,
                                     _i, _i, _i64, _p, _p, _p]),
    "sk_decode_step_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i, _i64, _i64, _i, _i]),
    "sk_decode_step_rescored_rows_offset": (_i64, [_i, _i, _i, _i, _i, _i, _i64, _i64, _i, _i]),
    "sk_decode_step": (_i, [C.POINTER(DecodeParams), _p]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library.  Raises if it has not been built (`python -m socket_b200.build`)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise SocketError(
                f"{LIB_PATH} is missing: build it with `python -m socket_b200.build` "
                "(there is no fallback implementation)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        l = lib()
        raise SocketError(f"{what}: {l.sk_status_string(status).decode()} — {l.sk_last_error().decode()}")


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def dtype_code(t: torch.Tensor) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise SocketError(f"unsupported dtype {t.dtype}") from None
