"""ctypes binding of the plain-C oracle (`oracle/c/socket_oracle.c`) and of the reference
scorer built by `oracle/build_oracle.py`.  TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np
import torch

from . import build_oracle

_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        path = build_oracle.C_LIB if os.path.exists(build_oracle.C_LIB) else build_oracle.build_c()
        _lib = C.CDLL(path)
        _lib.orc_list_len.restype = C.c_int64
        _lib.orc_list_len.argtypes = [C.c_int64, C.c_int, C.c_int, C.c_int64]
        _lib.orc_select_list.restype = C.c_int64
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def ref_lib():
    """The reference's scorer kernel compiled for the host, or None if it is not built."""
    global _ref
    if _ref is None:
        path = build_oracle.REF_LIB
        if not os.path.exists(path):
            path = build_oracle.build_ref()
        if path is None or not os.path.exists(path):
            return None
        _ref = C.CDLL(path)
    return _ref


def _p(t):
    if t is None:
        return C.c_void_p(0)
    if isinstance(t, np.ndarray):
        return C.c_void_p(t.ctypes.data)
    return C.c_void_p(t.data_ptr())


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(n))


def hash_keys(keys_nd: torch.Tensor, planes: torch.Tensor, exact: bool = True) -> torch.Tensor:
    keys_nd = keys_nd.contiguous()
    planes = planes.contiguous()
    L, P, D = planes.shape
    N = keys_nd.numel() // D
    codes = torch.empty(N, L, dtype=torch.int16)
    lib().orc_hash_keys(_p(keys_nd), C.c_int(_DT[keys_nd.dtype]), _p(planes),
                        C.c_int(_DT[planes.dtype]), C.c_int64(N), C.c_int(D), C.c_int(L),
                        C.c_int(P), C.c_int(int(exact)), _p(codes))
    return codes.view(*keys_nd.shape[:-1], L)


def value_norm(v: torch.Tensor) -> torch.Tensor:
    v = v.contiguous()
    D = v.shape[-1]
    N = v.numel() // D
    out = torch.empty(N, dtype=torch.float32)
    lib().orc_value_norm(_p(v), C.c_int(_DT[v.dtype]), C.c_int64(N), C.c_int(D), _p(out))
    return out.view(v.shape[:-1]).to(torch.float16)


def soft_hash(q_bhd, planes, protos_T, temperature: float = 1.0) -> torch.Tensor:
    q = q_bhd.contiguous()
    planes = planes.contiguous()
    protos = protos_T.float().contiguous()
    B, H, D = q.shape
    L, P, _ = planes.shape
    R = protos.shape[1]
    out = torch.empty(B, H, L, R, dtype=torch.float32)
    lib().orc_soft_hash(_p(q), C.c_int(_DT[q.dtype]), _p(planes), C.c_int(_DT[planes.dtype]),
                        _p(protos), C.c_int64(B * H), C.c_int(D), C.c_int(L), C.c_int(P),
                        C.c_int(R), C.c_float(temperature), _p(out))
    return out


def score(q_probs, codes_u8, v_norm_f16, T: int, allowed=None) -> torch.Tensor:
    """q_probs [B,H,L,R] f32, codes [B,Hkv,Tcap,L] u8, v_norm [B,Hkv,Tcap] f16 -> [B,H,T]."""
    q_probs = q_probs.float().contiguous()
    codes_u8 = codes_u8.contiguous()
    v_norm_f16 = v_norm_f16.contiguous()
    assert codes_u8.dtype == torch.uint8 and v_norm_f16.dtype == torch.float16
    B, H, L, R = q_probs.shape
    _, Hkv, Tcap, _ = codes_u8.shape
    out = torch.empty(B, H, T, dtype=torch.float32)
    al = None if allowed is None else allowed.to(torch.uint8).contiguous()
    lib().orc_score(_p(q_probs), _p(codes_u8), _p(v_norm_f16), _p(al), C.c_int(B), C.c_int(H),
                    C.c_int(Hkv), C.c_int64(T), C.c_int64(Tcap), C.c_int(L), C.c_int(R), _p(out))
    return out


def select_list(scores, sink: int, window: int, M: int, sorted_by_score: bool = False,
                allowed=None):
    scores = scores.float().contiguous()
    B, H, T = scores.shape
    Ktot = int(lib().orc_list_len(C.c_int64(T), C.c_int(sink), C.c_int(window), C.c_int64(M)))
    lst = torch.empty(B, H, Ktot, dtype=torch.int32)
    ln = torch.empty(B, H, dtype=torch.int32)
    al = None if allowed is None else allowed.to(torch.uint8).contiguous()
    lib().orc_select_list(_p(scores), _p(al), C.c_int64(B * H), C.c_int64(T), C.c_int(sink),
                          C.c_int(window), C.c_int64(M), C.c_int(int(sorted_by_score)),
                          _p(lst), _p(ln))
    return lst, ln


def sparse_attention(q, k, v, sparse_list, sparse_len, block_seq: int = 256) -> torch.Tensor:
    q = q.contiguous()
    k = k.contiguous()
    v = v.contiguous()
    sparse_list = sparse_list.contiguous()
    sparse_len = sparse_len.contiguous()
    B, H, D = q.shape
    _, Hkv, Tcap, _ = k.shape
    Ktot = sparse_list.shape[-1]
    out = torch.empty(B, H, D, dtype=torch.float32)
    lib().orc_sparse_attention(_p(q), C.c_int(_DT[q.dtype]), _p(k), _p(v), C.c_int(_DT[k.dtype]),
                               _p(sparse_list), _p(sparse_len), C.c_int(B), C.c_int(H),
                               C.c_int(Hkv), C.c_int64(Tcap), C.c_int(D), C.c_int64(Ktot),
                               C.c_int(block_seq), _p(out))
    return out


def ref_soft_hash_collision(q_probs_bh1lr, key_buckets_bhlt, allowed_bh1t, v_hist_bh1t):
    """Runs the reference's own kernel source on the host.  Argument layouts are the
    reference extension's (GPT-FAST/kernels/soft_hash_collision_loader.py:16-60)."""
    r = ref_lib()
    if r is None:
        raise RuntimeError("reference scorer not built (reference tree absent)")
    q = q_probs_bh1lr.float().contiguous()
    kb = key_buckets_bhlt.to(torch.int16).contiguous()
    al = allowed_bh1t.to(torch.bool).contiguous()
    vh = v_hist_bh1t.float().contiguous()
    B, H, _, L, R = q.shape
    T = kb.shape[-1]
    out = torch.zeros(B, H, 1, T, dtype=torch.float32)
    r.ref_soft_hash_collision(_p(q), _p(kb), _p(al), _p(vh), _p(out), C.c_int(B), C.c_int(H),
                              C.c_int(L), C.c_int(R), C.c_int(T))
    return out
