"""Tensor-level wrappers of the C-ABI entry points.

Each function checks what the reference checks at the same place (device, dtype, shape,
contiguity — `TORCH_CHECK`s of GPT-FAST/kernels/soft_hash_collision_loader.py:22-58 and the
asserts of GPT-FAST/kernels/sparse.py:29-35), allocates the outputs with torch and enqueues
the kernels on torch's current stream.  No function here synchronises with the host, and
none has a CPU path.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import check, dtype_code, lib, ptr, stream_ptr

_workspaces = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised scratch, one buffer per (device, stream), grown on demand.  The
    decode kernel leaves its ticket counters at zero, so the buffer is only cleared when
    it is (re)allocated."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("socket_b200 operators need CUDA tensors (there is no CPU path)")


def list_len(T: int, sink: int, window: int, M: int) -> int:
    return int(lib().sk_list_len(T, sink, window, M))


def hash_keys(keys: torch.Tensor, planes: torch.Tensor, code_dtype=torch.uint8) -> torch.Tensor:
    """keys [..., D] -> bucket codes [..., L] (uint8, or int16 like the reference)."""
    _require_cuda(keys, planes)
    L, P, D = planes.shape
    if keys.shape[-1] != D:
        raise RuntimeError(f"keys last dim {keys.shape[-1]} != planes head_dim {D}")
    keys = keys.contiguous()
    planes = planes.contiguous()
    N = keys.numel() // D
    code_bytes = {torch.uint8: 1, torch.int16: 2}[code_dtype]
    codes = torch.empty(*keys.shape[:-1], L, dtype=code_dtype, device=keys.device)
    check(lib().sk_hash_keys(ptr(keys), dtype_code(keys), D, ptr(planes), dtype_code(planes), N, D, L,
                             P, ptr(codes), code_bytes, L, stream_ptr(keys.device)), "sk_hash_keys")
    return codes


def hash_keys_tc(keys: torch.Tensor, planes: torch.Tensor, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Tensor-core bulk hashing: bf16 keys [..., 128], planes [32, 8, 128] -> uint8 codes [..., 32],
    bit-identical to `hash_keys`.  `status` (int32 device word) collects device-side flags."""
    _require_cuda(keys, planes)
    L, P, D = planes.shape
    keys = keys.contiguous()
    planes = planes.contiguous()
    N = keys.numel() // D
    codes = torch.empty(*keys.shape[:-1], L, dtype=torch.uint8, device=keys.device)
    ws = torch.empty(int(lib().sk_hash_keys_tc_workspace_bytes(N)), dtype=torch.uint8, device=keys.device)
    if dtype_code(keys) != _lib.SK_BF16 or dtype_code(planes) != _lib.SK_BF16:
        raise RuntimeError("hash_keys_tc needs bf16 keys and planes")
    check(lib().sk_hash_keys_tc(ptr(keys), D, ptr(planes), N, D, L, P, ptr(codes), L, None, ptr(ws), ws.numel(),
                                ptr(status), stream_ptr(keys.device)), "sk_hash_keys_tc")
    return codes


TC_APPEND_MIN_ROWS = 1024


def kv_append(k_cache, v_cache, codes, v_norm, prefill_len, input_pos, k_new, v_new, planes,
              status: Optional[torch.Tensor] = None) -> None:
    """Write S new tokens (k_new/v_new [B,S,Hkv,D]) at `input_pos` [S] (int64, device) into
    the cache tensors, with their bucket codes and value norms."""
    _require_cuda(k_cache, v_cache, codes, v_norm, prefill_len, input_pos, k_new, v_new, planes)
    B, Hkv, Tcap, D = k_cache.shape
    L, P, _ = planes.shape
    S = k_new.shape[1]
    assert k_new.shape == (B, S, Hkv, D) and v_new.shape == (B, S, Hkv, D)
    assert input_pos.dtype == torch.int64 and input_pos.numel() == S
    assert codes.dtype == torch.uint8 and codes.shape == (B, Hkv, Tcap, L)
    assert v_norm.dtype == torch.float16 and v_norm.shape == (B, Hkv, Tcap)
    assert k_new.dtype == k_cache.dtype == v_cache.dtype == v_new.dtype
    for t in (k_cache, v_cache, codes, v_norm):
        assert t.is_contiguous()
    k_new = k_new.contiguous()
    v_new = v_new.contiguous()
    planes = planes.contiguous()
    if (B * S * Hkv >= TC_APPEND_MIN_ROWS and k_new.dtype == torch.bfloat16 and planes.dtype == torch.bfloat16
            and D == 128 and L == 32 and P == 8):
        # prefill-sized batch: projection on the tensor cores
        ws = torch.empty(int(lib().sk_kv_append_tc_workspace_bytes(B, S, Hkv)), dtype=torch.uint8,
                         device=k_cache.device)
        check(lib().sk_kv_append_tc(ptr(k_new), ptr(v_new), dtype_code(k_new), ptr(input_pos), ptr(planes),
                                    dtype_code(planes), ptr(k_cache), ptr(v_cache), ptr(codes), ptr(v_norm),
                                    ptr(prefill_len), ptr(status), B, S, Hkv, D, Tcap, L, P, ptr(ws), ws.numel(),
                                    stream_ptr(k_cache.device)), "sk_kv_append_tc")
        return
    check(lib().sk_kv_append(ptr(k_new), ptr(v_new), dtype_code(k_new), ptr(input_pos), ptr(planes),
                             dtype_code(planes), ptr(k_cache), ptr(v_cache), ptr(codes), ptr(v_norm),
                             ptr(prefill_len), ptr(status), B, S, Hkv, D, Tcap, L, P,
                             stream_ptr(k_cache.device)), "sk_kv_append")


def rope_split(qkv: torch.Tensor, freqs_cis: torch.Tensor, input_pos: torch.Tensor, n_head: int,
               n_kv_heads: int, q_out: torch.Tensor, k_out: torch.Tensor, v_out: torch.Tensor,
               status: Optional[torch.Tensor] = None) -> None:
    """qkv [B,1,(H+2Hkv)*D] of one new token -> q_out [B,H,D], k_out / v_out [B,1,Hkv,D], q and k
    rotated by the angles of position `input_pos[0]` (device int64); freqs_cis [n_pos, D/2, 2]."""
    _require_cuda(qkv, freqs_cis, input_pos, q_out, k_out, v_out)
    B, H, D = q_out.shape
    assert H == n_head and k_out.shape == (B, 1, n_kv_heads, D) and v_out.shape == k_out.shape
    assert qkv.is_contiguous() and qkv.numel() == B * (H + 2 * n_kv_heads) * D
    assert q_out.is_contiguous() and k_out.is_contiguous() and v_out.is_contiguous()
    assert freqs_cis.is_contiguous() and freqs_cis.shape[1:] == (D // 2, 2)
    assert input_pos.dtype == torch.int64
    check(lib().sk_rope_split(ptr(qkv), dtype_code(qkv), ptr(freqs_cis), dtype_code(freqs_cis), ptr(input_pos), B, H,
                              n_kv_heads, D, freqs_cis.shape[0], ptr(q_out), ptr(k_out), ptr(v_out), ptr(status),
                              stream_ptr(qkv.device)), "sk_rope_split")


def soft_hash(q_bhd: torch.Tensor, planes: torch.Tensor, protos_T: torch.Tensor,
              temperature: float = 1.0, n_kv_heads: Optional[int] = None,
              want_probs: bool = True, want_lut: bool = False):
    """q [B,H,D] -> (q_probs [B,H,L,R] fp32 or None, scorer table or None)."""
    _require_cuda(q_bhd, planes, protos_T)
    B, H, D = q_bhd.shape
    L, P, D2 = planes.shape
    assert D2 == D
    R = protos_T.shape[1]
    assert protos_T.shape[0] == P
    Hkv = n_kv_heads if n_kv_heads is not None else H
    q = q_bhd.contiguous()
    planes = planes.contiguous()
    protos = protos_T.to(torch.float32).contiguous()
    probs = torch.empty(B, H, L, R, dtype=torch.float32, device=q.device) if want_probs else None
    lut = torch.empty(B * H * L * R, dtype=torch.float32, device=q.device) if want_lut else None
    check(lib().sk_soft_hash(ptr(q), dtype_code(q), ptr(planes), dtype_code(planes), ptr(protos),
                             float(temperature), B, H, Hkv, D, L, P, R, ptr(probs), ptr(lut),
                             stream_ptr(q.device)), "sk_soft_hash")
    return probs, lut


def lut_from_probs(q_probs: torch.Tensor, n_kv_heads: int) -> torch.Tensor:
    _require_cuda(q_probs)
    B, H, L, R = q_probs.shape
    q_probs = q_probs.contiguous()
    lut = torch.empty(B * H * L * R, dtype=torch.float32, device=q_probs.device)
    check(lib().sk_lut_from_probs(ptr(q_probs), dtype_code(q_probs), B, H, n_kv_heads, L, R, ptr(lut),
                                  stream_ptr(q_probs.device)), "sk_lut_from_probs")
    return lut


def score(lut: torch.Tensor, codes: torch.Tensor, v_norm: torch.Tensor, n_heads: int, T: int,
          R: int = 256, allowed: Optional[torch.Tensor] = None,
          T_dev: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
          status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """codes [B,Hkv,Tcap,L] uint8, v_norm [B,Hkv,Tcap] fp16 -> scores [B,H,T] fp32."""
    _require_cuda(lut, codes, v_norm, allowed)
    B, Hkv, Tcap, L = codes.shape
    assert codes.dtype == torch.uint8 and codes.is_contiguous()
    assert v_norm.dtype == torch.float16 and v_norm.is_contiguous() and v_norm.shape == (B, Hkv, Tcap)
    if allowed is not None:
        assert allowed.shape == (B, n_heads, T)
        allowed = allowed.to(torch.uint8).contiguous() if allowed.dtype != torch.uint8 else allowed.contiguous()
    if out is None:
        out = torch.empty(B, n_heads, T, dtype=torch.float32, device=codes.device)
    assert out.dtype == torch.float32 and out.stride(2) == 1 and out.stride(0) == n_heads * out.stride(1)
    check(lib().sk_score(ptr(lut), ptr(codes), ptr(v_norm), ptr(allowed), B, n_heads, Hkv, L, R, T,
                         ptr(T_dev), Tcap, ptr(out), out.stride(1), ptr(status),
                         stream_ptr(codes.device)), "sk_score")
    return out


def soft_hash_collision(q_probs: torch.Tensor, key_buckets: torch.Tensor, allowed_ext: torch.Tensor,
                        v_hist: torch.Tensor) -> torch.Tensor:
    """Same call as the reference's scorer extension
    (GPT-FAST/kernels/soft_hash_collision_loader.py:16-72): q_probs [B,H,1,L,R] fp32,
    key_buckets [B,H,L,T] int16, allowed_ext [B,H,1,T] bool, v_hist [B,H,1,T] fp32 ->
    [B,H,1,T] fp32.  Same checks, same RuntimeError on violation."""
    for name, t in (("q_probs", q_probs), ("key_buckets", key_buckets),
                    ("allowed_ext", allowed_ext), ("v_hist", v_hist)):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be CUDA")
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    if q_probs.dtype != torch.float32:
        raise RuntimeError("q_probs must be float32")
    if key_buckets.dtype != torch.int16:
        raise RuntimeError("key_buckets must be int16")
    if allowed_ext.dtype != torch.bool:
        raise RuntimeError("allowed_ext must be bool")
    if v_hist.dtype != torch.float32:
        raise RuntimeError("v_hist must be float32")
    if q_probs.dim() != 5:
        raise RuntimeError("q_probs must be [B,H,1,L,R]")
    if key_buckets.dim() != 4:
        raise RuntimeError("key_buckets must be [B,H,L,T_k]")
    if allowed_ext.dim() != 4:
        raise RuntimeError("allowed_ext must be [B,H,1,T_k]")
    if v_hist.dim() != 4:
        raise RuntimeError("v_hist must be [B,H,1,T_k]")
    B, H, _, L, R = q_probs.shape
    T = key_buckets.shape[3]
    if tuple(key_buckets.shape[:3]) != (B, H, L):
        raise RuntimeError("key_buckets shape mismatch")
    if tuple(allowed_ext.shape) != (B, H, 1, T):
        raise RuntimeError("allowed_ext shape mismatch")
    if tuple(v_hist.shape) != (B, H, 1, T):
        raise RuntimeError("v_hist shape mismatch")
    out = torch.empty(B, H, 1, T, dtype=torch.float32, device=q_probs.device)
    check(lib().sk_score_compat(ptr(q_probs), ptr(key_buckets), ptr(allowed_ext), ptr(v_hist), ptr(out),
                                B, H, L, R, T, stream_ptr(q_probs.device)), "sk_score_compat")
    return out


def select_list(scores: torch.Tensor, T: int, M: int, sink: int, window: int,
                sorted_by_score: bool = False, allowed: Optional[torch.Tensor] = None,
                T_dev: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """scores [B,H,>=T] fp32 -> (sparse_list int32 [B,H,Ktot], sparse_len int32 [B,H])."""
    _require_cuda(scores, allowed)
    B, H = scores.shape[:2]
    assert scores.dtype == torch.float32 and scores.stride(2) == 1
    assert scores.stride(0) == H * scores.stride(1)
    if allowed is not None:
        assert allowed.shape == (B, H, T)
        allowed = allowed.to(torch.uint8).contiguous() if allowed.dtype != torch.uint8 else allowed.contiguous()
    Ktot = list_len(T, sink, window, M)
    lst = torch.empty(B, H, Ktot, dtype=torch.int32, device=scores.device)
    ln = torch.empty(B, H, dtype=torch.int32, device=scores.device)
    check(lib().sk_select_list(ptr(scores), scores.stride(1), ptr(allowed), B * H, T, ptr(T_dev), M, sink,
                               window, int(sorted_by_score), ptr(lst), Ktot, ptr(ln), 0,
                               stream_ptr(scores.device)), "sk_select_list")
    return lst, ln


def score_select_applicable(B: int, H: int, Hkv: int, L: int, R: int, T: int, M: int) -> bool:
    return bool(lib().sk_score_select_applicable(B, H, Hkv, L, R, T, M))


def score_select_list(lut: torch.Tensor, codes: torch.Tensor, v_norm: torch.Tensor, n_heads: int, T: int,
                      M: int, sink: int, window: int, R: int = 256,
                      T_dev: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None):
    """Fused scorer + select (`sk_score_select_list`): the list of `score` followed by
    `select_list`, without the score array.  Returns (sparse_list, sparse_len, workspace); the
    first int32 of the workspace counts the rows that had to be rescored so far."""
    _require_cuda(lut, codes, v_norm)
    B, Hkv, Tcap, L = codes.shape
    M = min(M, T)
    Ktot = list_len(T, sink, window, M)
    lst = torch.empty(B, n_heads, Ktot, dtype=torch.int32, device=codes.device)
    ln = torch.empty(B, n_heads, dtype=torch.int32, device=codes.device)
    need = int(lib().sk_score_select_workspace_bytes(B, n_heads, Hkv, L, T, M))
    if workspace is None or workspace.numel() < need:
        workspace = torch.zeros(need, dtype=torch.uint8, device=codes.device)
    check(lib().sk_score_select_list(ptr(lut), ptr(codes), ptr(v_norm), B, n_heads, Hkv, L, R, T, ptr(T_dev),
                                     Tcap, M, sink, window, ptr(lst), Ktot, ptr(ln), ptr(workspace),
                                     workspace.numel(), None, stream_ptr(codes.device)),
          "sk_score_select_list")
    return lst, ln, workspace


def packed_applicable(B: int, H: int, Hkv: int, L: int, R: int, T: int, M: int) -> bool:
    return bool(lib().sk_packed_applicable(B, H, Hkv, L, R, T, M))


def packed_preferred(B: int, H: int, Hkv: int, L: int, R: int, T: int, M: int) -> bool:
    """Whether `sk_decode_step` takes the packed scan for this shape on its own."""
    return bool(lib().sk_packed_preferred(B, H, Hkv, L, R, T, M))


def soft_hash_packed(q_bhd: torch.Tensor, planes: torch.Tensor, protos_T: torch.Tensor,
                     temperature: float = 1.0, n_kv_heads: Optional[int] = None):
    """q [B,H,D] -> (fp32 scorer table, packed 12-bit copy of it) for `score_select_packed`
    (`sk_soft_hash_packed`)."""
    _require_cuda(q_bhd, planes, protos_T)
    B, H, D = q_bhd.shape
    L, P, _ = planes.shape
    R = protos_T.shape[1]
    Hkv = n_kv_heads if n_kv_heads is not None else H
    q = q_bhd.contiguous()
    planes = planes.contiguous()
    protos = protos_T.to(torch.float32).contiguous()
    lut = torch.empty(B * H * L * R, dtype=torch.float32, device=q.device)
    nbytes = int(lib().sk_packed_table_bytes(B, H, Hkv))
    if nbytes == 0:
        raise RuntimeError("soft_hash_packed: needs a multiple of 4 query heads per KV head")
    packed = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    check(lib().sk_soft_hash_packed(ptr(q), dtype_code(q), ptr(planes), dtype_code(planes), ptr(protos),
                                    float(temperature), B, H, Hkv, D, L, P, R, ptr(lut), ptr(packed),
                                    stream_ptr(q.device)), "sk_soft_hash_packed")
    return lut, packed


def score_select_packed(lut: torch.Tensor, packed: torch.Tensor, codes: torch.Tensor, v_norm: torch.Tensor,
                        n_heads: int, T: int, M: int, sink: int, window: int, R: int = 256,
                        T_dev: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None,
                        stages: int = 3, out=None):
    """The fused scorer + select on the packed table (`sk_score_select_packed`); same result as
    `score_select_list`.  Returns (sparse_list, sparse_len, workspace)."""
    _require_cuda(lut, packed, codes, v_norm)
    B, Hkv, Tcap, L = codes.shape
    M = min(M, T)
    Ktot = list_len(T, sink, window, M)
    if out is None:
        lst = torch.empty(B, n_heads, Ktot, dtype=torch.int32, device=codes.device)
        ln = torch.empty(B, n_heads, dtype=torch.int32, device=codes.device)
    else:
        lst, ln = out
    need = int(lib().sk_score_select_workspace_bytes(B, n_heads, Hkv, L, T, M))
    if workspace is None or workspace.numel() < need:
        workspace = torch.zeros(need, dtype=torch.uint8, device=codes.device)
    check(lib().sk_score_select_packed(ptr(lut), ptr(packed), ptr(codes), ptr(v_norm), B, n_heads, Hkv, L, R, T,
                                       ptr(T_dev), Tcap, M, sink, window, ptr(lst), Ktot, ptr(ln),
                                       ptr(workspace), workspace.numel(), None, stages, stream_ptr(codes.device)),
          "sk_score_select_packed")
    return lst, ln, workspace


def score_select_cluster_size(B: int, H: int, Hkv: int, L: int, R: int, T: int, M: int) -> int:
    """Cluster size (2..16) of the one-launch scorer + select for this shape on the current
    device, 0 when the shape is outside it."""
    return int(lib().sk_score_select_cluster_size(B, H, Hkv, L, R, T, M))


def score_select_cluster(lut: torch.Tensor, codes: torch.Tensor, v_norm: torch.Tensor, n_heads: int, T: int,
                         M: int, sink: int, window: int, R: int = 256, T_dev: Optional[torch.Tensor] = None,
                         status: Optional[torch.Tensor] = None):
    """Scorer + exact select in one launch on thread-block clusters (`sk_score_select_cluster`):
    the list of `score` followed by `select_list`, scores never leave the chip.  Returns
    (sparse_list, sparse_len)."""
    _require_cuda(lut, codes, v_norm)
    B, Hkv, Tcap, L = codes.shape
    M = min(M, T)
    Ktot = list_len(T, sink, window, M)
    lst = torch.empty(B, n_heads, Ktot, dtype=torch.int32, device=codes.device)
    ln = torch.empty(B, n_heads, dtype=torch.int32, device=codes.device)
    check(lib().sk_score_select_cluster(ptr(lut), ptr(codes), ptr(v_norm), B, n_heads, Hkv, L, R, T, ptr(T_dev),
                                        Tcap, M, sink, window, ptr(lst), Ktot, ptr(ln), ptr(status),
                                        stream_ptr(codes.device)), "sk_score_select_cluster")
    return lst, ln


def sparse_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  sparse_list: torch.Tensor, sparse_len: torch.Tensor, T: Optional[int] = None,
                  T_dev: Optional[torch.Tensor] = None,
                  status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [B,H,D]; k_cache/v_cache [B,Hkv,Tcap,D] (any strides with a unit last stride) ->
    out [B,H,D] in q's dtype."""
    _require_cuda(q, k_cache, v_cache, sparse_list, sparse_len)
    B, H, D = q.shape
    Hkv = k_cache.shape[1]
    assert k_cache.shape == v_cache.shape and k_cache.stride() == v_cache.stride()
    assert k_cache.stride(3) == 1 and k_cache.dtype == v_cache.dtype
    assert sparse_list.dtype == torch.int32 and sparse_len.dtype == torch.int32
    assert sparse_list.shape[:2] == (B, H) and sparse_len.shape == (B, H)
    q = q.contiguous()
    sparse_list = sparse_list.contiguous()
    sparse_len = sparse_len.contiguous()
    Kmax = sparse_list.shape[2]
    if T is None:
        T = k_cache.shape[2]
    out = torch.empty(B, H, D, dtype=q.dtype, device=q.device)
    if Kmax == 0:
        return out.zero_()
    need = int(lib().sk_sparse_decode_workspace_bytes(B, H, D, Kmax))
    ws = _workspace(q.device, need)
    check(lib().sk_sparse_decode(ptr(q), dtype_code(q), ptr(k_cache), ptr(v_cache), dtype_code(k_cache),
                                 k_cache.stride(0), k_cache.stride(1), k_cache.stride(2),
                                 ptr(sparse_list), Kmax, ptr(sparse_len), Kmax, ptr(out), B, H, Hkv, D, T,
                                 ptr(T_dev), ptr(ws), ws.numel(), ptr(status), stream_ptr(q.device)),
          "sk_sparse_decode")
    return out


# sk_select_path: how the decode step builds its list (all paths give the same list)
SELECT_PATHS = {"auto": 0, "two_launch": 1, "filter": 2, "cluster": 3, "filter_f32": 4, "filter_packed": 5}


class DecodeStep:
    """One fused decode step of one layer (`sk_decode_step`): append+hash the new token,
    soft-hash the query, score, select, attend — four launches on the current stream, no
    host synchronisation, so it can be captured in a CUDA graph.  Holds the parameter
    block and the scratch memory; `run()` re-enqueues the step on whatever the tensors
    given at construction contain at that moment."""

    def __init__(self, cache, q: torch.Tensor, k_new: Optional[torch.Tensor],
                 v_new: Optional[torch.Tensor], input_pos: Optional[torch.Tensor],
                 planes: torch.Tensor, protos_T: torch.Tensor, out: torch.Tensor, *, topk: int,
                 sink: int, window: int, T_max: int, temperature: float = 1.0,
                 keep_list: bool = False, select_path: str = "auto"):
        B, Hkv, Tcap, D = cache.k_cache.shape
        H = q.shape[1]
        L, P, _ = planes.shape
        R = protos_T.shape[1]
        dev = q.device
        self._keep = (cache, q, k_new, v_new, input_pos, planes, protos_T, out)
        self.protos = protos_T.to(torch.float32).contiguous()
        nbytes = int(lib().sk_decode_step_workspace_bytes(B, H, Hkv, D, L, R, T_max, topk, sink, window))
        self.workspace = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.list = self.list_len = None
        ktot = list_len(T_max, sink, window, topk)
        if keep_list:
            self.list = torch.full((B, H, ktot), -1, dtype=torch.int32, device=dev)
            self.list_len = torch.zeros(B, H, dtype=torch.int32, device=dev)
        p = _lib.DecodeParams()
        p.q, p.k_new, p.v_new, p.input_pos = ptr(q), ptr(k_new), ptr(v_new), ptr(input_pos)
        p.planes, p.protos_T, p.temperature = ptr(planes), ptr(self.protos), float(temperature)
        p.k_cache, p.v_cache = ptr(cache.k_cache), ptr(cache.v_cache)
        p.codes, p.v_norm, p.prefill_len = ptr(cache.k_hard), ptr(cache.v_norm), ptr(cache.prefill_len)
        p.out, p.list, p.list_len, p.list_row_stride = ptr(out), ptr(self.list), ptr(self.list_len), ktot
        p.workspace, p.workspace_bytes, p.status = ptr(self.workspace), nbytes, ptr(self.status)
        p.q_dtype, p.kv_dtype, p.plane_dtype = dtype_code(q), dtype_code(cache.k_cache), dtype_code(planes)
        p.B, p.H, p.Hkv, p.D, p.L, p.P, p.R = B, H, Hkv, D, L, P, R
        p.Tcap, p.T_max, p.M, p.sink, p.window = Tcap, T_max, topk, sink, window
        p.select_path = SELECT_PATHS[select_path]
        self.params = p
        self.device = dev
        self._topk_max = topk
        # prologue (append + soft hash in one launch when q and the cache share a dtype), score,
        # select, decode
        self.n_launches = 4 if (k_new is None or q.dtype == cache.k_cache.dtype) else 5
        fused = bool(lib().sk_score_select_applicable(B, H, Hkv, L, R, T_max, topk))
        cluster = bool(lib().sk_score_select_cluster_size(B, H, Hkv, L, R, T_max, topk))
        if select_path == "cluster" or (select_path == "auto" and cluster and not fused):
            self.n_launches -= 1          # scorer and select are one launch

        self._rescored_off = int(lib().sk_decode_step_rescored_rows_offset(B, H, Hkv, D, L, R, T_max, topk,
                                                                           sink, window))

    def set_topk(self, topk: int) -> None:
        """Another top-k budget for the following runs (at most the budget given at construction,
        which sized the kept list).  The scratch layout follows the budget, so the workspace grows
        if this budget's layout needs more; the select counters restart.  For eager callers whose
        budget is a fraction of the live length (the reference's `_effective_size`,
        pipeline/train_quest/modeling/modeling_llama.py:645-648); a captured CUDA graph keeps the
        budget it was captured with."""
        p = self.params
        assert 0 <= topk <= self._topk_max, "budget above the one the step was built for"
        if topk == p.M:
            return
        nbytes = int(lib().sk_decode_step_workspace_bytes(p.B, p.H, p.Hkv, p.D, p.L, p.R, p.T_max, topk,
                                                          p.sink, p.window))
        if nbytes > self.workspace.numel():
            self.workspace = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        p.workspace, p.workspace_bytes = ptr(self.workspace), self.workspace.numel()
        p.M = topk
        # The decode kernel's ticket counters sit at the start of every layout and are left at zero by
        # every call; everything else is rewritten by each step except the select counters.
        self._rescored_off = int(lib().sk_decode_step_rescored_rows_offset(p.B, p.H, p.Hkv, p.D, p.L, p.R, p.T_max,
                                                                           topk, p.sink, p.window))
        if self._rescored_off >= 0:
            self.workspace[self._rescored_off:self._rescored_off + 256].zero_()

    def rebind(self, q: torch.Tensor, k_new: Optional[torch.Tensor], v_new: Optional[torch.Tensor],
               input_pos: Optional[torch.Tensor], out: torch.Tensor) -> None:
        """Point the step at other input/output tensors of the same shapes and dtypes; the
        scratch memory is kept.  (A CUDA graph captured before this call still holds the old
        addresses.)"""
        old_q, old_out = self._keep[1], self._keep[7]
        assert q.shape == old_q.shape and q.dtype == old_q.dtype and out.shape == old_out.shape
        assert q.is_contiguous() and out.is_contiguous()
        assert (k_new is None) == (self._keep[2] is None)
        if k_new is not None:
            assert k_new.is_contiguous() and v_new.is_contiguous()
            assert k_new.shape == self._keep[2].shape and k_new.dtype == self._keep[2].dtype
        self._keep = (self._keep[0], q, k_new, v_new, input_pos) + self._keep[5:7] + (out,)
        p = self.params
        p.q, p.k_new, p.v_new, p.input_pos, p.out = ptr(q), ptr(k_new), ptr(v_new), ptr(input_pos), ptr(out)

    def run(self) -> None:
        check(lib().sk_decode_step(C.byref(self.params), stream_ptr(self.device)), "sk_decode_step")

    def rescored_rows(self) -> Optional[int]:
        """Rows that went through the select kernel's full rescoring path in the steps run so far
        (None if this shape's path keeps no count).  Synchronises."""
        if self._rescored_off < 0:
            return None
        return int(self.workspace[self._rescored_off:self._rescored_off + 4].view(torch.int32).item())

    def select_stats(self) -> Optional[dict]:
        """Counters of the candidate select over the steps run so far: rows rescored in full, keys
        scored exactly inside the k-th score's bracket (packed table only), rows whose bracket was
        large enough to be ranked by the radix pass.  Synchronises."""
        if self._rescored_off < 0:
            return None
        c = self.workspace[self._rescored_off:self._rescored_off + 36].view(torch.int32).tolist()
        return {"rescored_rows": c[0], "bracket_keys": c[1], "bracket_rows_radix": c[2],
                "rescored_run_overflow": c[3], "rescored_candidate_count": c[4], "rescored_unproved": c[5],
                # why a packed row was unproved: its bracket reached below the largest cut / held too many keys
                "unproved_below_cut": c[6], "unproved_bracket_size": c[7], "unproved_counts": c[8]}
