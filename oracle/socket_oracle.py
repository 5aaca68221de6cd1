"""CPU oracle for the SOCKET sparse-attention decode path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch-on-CPU / numpy arithmetic, what the reference
computes on the path  hash keys -> soft-hash query -> score keys -> top-k + sink/window
list -> sparse attention.  Nothing in the shipped package imports it: only the tests, the
smoke check and the benchmark's CPU-baseline leg do, and only as the checker.

Pinning: the reference ships no tests and no golden vectors for this path.  The oracle is
pinned instead against outputs of the reference's own code executed on CPU
(`tests/golden/make_golden.py` runs `Attention.hard_hash_keys/soft_hash`, the reference
scorer kernel text compiled as C++, the reference list-assembly code and its Triton
decode kernels under the Triton interpreter, and freezes the results as fixtures);
`tests/test_oracle_golden.py` checks every function here against those fixtures.

Each function cites the reference lines it follows (paths relative to the reference root).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch


# --------------------------------------------------------------------------------------
# hashing
# --------------------------------------------------------------------------------------
def pack_bits(bits: torch.Tensor) -> torch.Tensor:
    """bits [..., P] (bool) -> int16 code, first plane = most significant bit.
    Follows GPT-FAST/model.py:403-407."""
    P = bits.shape[-1]
    code = torch.zeros(bits.shape[:-1], dtype=torch.int32)
    for p in range(P):
        code = code * 2 + bits[..., p].to(torch.int32)
    return code.to(torch.int16)


def hard_hash_keys(keys_bshd: torch.Tensor, planes: torch.Tensor) -> torch.Tensor:
    """keys [B,S,Hkv,D], planes [L,P,D] -> int16 codes [B,S,Hkv,L].
    Sign-random-projection: bit = (<key, plane> >= 0); follows GPT-FAST/model.py:409-413.
    Computed in the dtype of the inputs promoted to fp32 (what the reference does on CPU
    for fp32 tensors)."""
    proj = torch.einsum("bshd,lpd->bshlp", keys_bshd.float(), planes.float())
    return pack_bits(proj >= 0)


def hard_hash_keys_exact(keys_bshd: torch.Tensor, planes: torch.Tensor,
                         band: float = 2.0 ** -20) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp64 arbiter for the hash bits.  Returns (codes int16 [B,S,Hkv,L],
    ambiguous bool [B,S,Hkv,L,P]).  A projection is *ambiguous* when
    |<k,p>| <= band * sum_d |k_d p_d|: there a different fp32 summation order may flip
    the sign, so a comparison against an fp32 implementation must skip those bits.  For
    bf16/fp16 inputs every product is exact in fp64 and the fp64 sum decides the true
    sign."""
    k = keys_bshd.double()
    p = planes.double()
    proj = torch.einsum("bshd,lpd->bshlp", k, p)
    mag = torch.einsum("bshd,lpd->bshlp", k.abs(), p.abs())
    return pack_bits(proj >= 0), proj.abs() <= band * mag


def value_norm(v_bshd: torch.Tensor) -> torch.Tensor:
    """||v||_2 computed in fp32 and stored as fp16; follows GPT-FAST/model.py:450."""
    return torch.linalg.vector_norm(v_bshd.float(), ord=2, dim=-1).to(torch.float16)


def soft_hash(q_bhd: torch.Tensor, planes: torch.Tensor, protos_T: torch.Tensor,
              temperature: float = 1.0) -> torch.Tensor:
    """q [B,H,D] -> q_probs [B,H,L,R]: per table a softmax over the R buckets of
    (tanh(<q, plane_p>)/sqrt(D)) . protos_T.  Follows GPT-FAST/model.py:392-401; the
    HuggingFace variant additionally divides the logits by a temperature
    (pipeline/train_quest/modeling/modeling_llama.py:638), exposed here as
    ``temperature`` (1.0 = the GPT-FAST formula)."""
    q = q_bhd.float()
    D = q.shape[-1]
    proj = torch.einsum("bhd,lpd->bhlp", q, planes.float())
    t = torch.tanh(proj) / max(math.sqrt(D), 1e-6)
    logits = torch.einsum("bhlp,pr->bhlr", t, protos_T.float())
    if temperature != 1.0:
        logits = logits / temperature
    return torch.softmax(logits, dim=-1)


# --------------------------------------------------------------------------------------
# layout glue of the caller
# --------------------------------------------------------------------------------------
def relayout_for_reference(k_hard_bhtl: torch.Tensor, v_norm_bht: torch.Tensor, rep: int):
    """[B,Hkv,T,L] codes / [B,Hkv,T] norms -> the query-head-expanded, table-major layout
    the reference scorer consumes: codes [B,H,L,T], norms [B,H,T].
    Follows GPT-FAST/model.py:494-506."""
    kh = k_hard_bhtl.repeat_interleave(rep, dim=1) if rep != 1 else k_hard_bhtl
    kh = kh.permute(0, 1, 3, 2).contiguous()
    vn = v_norm_bht.repeat_interleave(rep, dim=1) if rep != 1 else v_norm_bht
    return kh, vn


# --------------------------------------------------------------------------------------
# scorer
# --------------------------------------------------------------------------------------
def soft_hash_collision(q_probs: torch.Tensor, key_buckets_bhlt: torch.Tensor,
                        allowed_bht: torch.Tensor, v_hist_bht: torch.Tensor) -> torch.Tensor:
    """score[b,h,t] = allowed ? (sum_{l=0..L-1} q_probs[b,h,l,code[b,h,l,t]]) * v_hist : -inf.
    fp32, tables added in ascending order starting from 0.0 — the order of
    GPT-FAST/kernels/soft_hash_collision.cu:45-53."""
    B, H, L, R = q_probs.shape
    T = key_buckets_bhlt.shape[-1]
    qp = q_probs.float().contiguous().numpy()
    codes = key_buckets_bhlt.numpy().astype(np.int64)
    acc = np.zeros((B, H, T), dtype=np.float32)
    for l in range(L):
        acc = acc + np.take_along_axis(qp[:, :, l, :], codes[:, :, l, :], axis=-1)
    out = acc * v_hist_bht.float().numpy()
    out = np.where(allowed_bht.numpy(), out, np.float32(-np.inf)).astype(np.float32)
    return torch.from_numpy(out)


def score_keys_native(q_probs: torch.Tensor, codes_bhtl: torch.Tensor,
                      v_norm_bht: torch.Tensor, allowed_bht: Optional[torch.Tensor] = None):
    """Same score from the cache-native layout (codes [B,Hkv,T,L], norms [B,Hkv,T] fp16):
    the composition of `relayout_for_reference`, the `.float()` casts of
    GPT-FAST/kernels/sparse.py:42-48 and `soft_hash_collision`."""
    B, H, L, R = q_probs.shape
    rep = H // codes_bhtl.shape[1]
    kh, vn = relayout_for_reference(codes_bhtl.to(torch.int16), v_norm_bht, rep)
    T = kh.shape[-1]
    if allowed_bht is None:
        allowed_bht = torch.ones(B, H, T, dtype=torch.bool)
    return soft_hash_collision(q_probs, kh, allowed_bht, vn.float())


# --------------------------------------------------------------------------------------
# selection + list assembly
# --------------------------------------------------------------------------------------
def topk_lowest_index(scores_row: np.ndarray, k: int) -> np.ndarray:
    """Indices of the k largest scores of one row; among equal scores the smallest index
    wins.  Returned in ascending index order.  (`torch.topk`, GPT-FAST/kernels/sparse.py:57,
    leaves the choice among equal scores unspecified; this is the deterministic rule the
    CUDA select implements.)"""
    order = np.lexsort((np.arange(scores_row.shape[0]), -scores_row.astype(np.float64)))
    return np.sort(order[:k]).astype(np.int32)


def check_topk_set(scores_row: np.ndarray, chosen: np.ndarray, k: int) -> None:
    """Assert that ``chosen`` is a valid top-k index set of ``scores_row`` with ties at
    the k-th value resolved towards the smallest indices."""
    T = scores_row.shape[0]
    k = min(k, T)
    chosen = np.asarray(chosen)
    assert chosen.shape[0] == k, (chosen.shape, k)
    assert len(set(chosen.tolist())) == k, "duplicate index in top-k"
    if k == 0:
        return
    assert chosen.min() >= 0 and chosen.max() < T
    kth = np.sort(scores_row)[::-1][k - 1]
    greater = np.nonzero(scores_row > kth)[0]
    assert set(greater.tolist()) <= set(chosen.tolist()), "a strictly greater score is missing"
    ties = np.nonzero(scores_row == kth)[0]
    need = k - greater.shape[0]
    assert set(ties[:need].tolist()) <= set(chosen.tolist()), "tie not resolved to lowest index"


def base_indices(T: int, sink: int, window: int) -> np.ndarray:
    """Structured part of the list: [0..sink) ++ [max(T-window, sink)..T), or [T-1] when
    both are empty.  Follows GPT-FAST/kernels/sparse.py:70-84."""
    sink = max(0, min(sink, T))
    window = max(0, min(window, T))
    parts = []
    if sink > 0:
        parts.append(np.arange(sink, dtype=np.int32))
    if window > 0:
        start = max(T - window, sink)
        if start < T:
            parts.append(np.arange(start, T, dtype=np.int32))
    if not parts:
        return np.array([T - 1], dtype=np.int32)
    return np.concatenate(parts)


def build_sparse_list_decode(q_probs, k_hard_bhlt, v_norm_bht, allowed_bht,
                             sink: int, window: int, M: int, sorted_by_score: bool = True):
    """(sparse_list int32 [B,H,Ktot], sparse_len int32 [B,H], scores fp32 [B,H,T]).

    Follows GPT-FAST/kernels/sparse.py:39-95: scores from the collision kernel, top-M
    indices, entries that are out of range or not allowed become -1, then
    ``[sink..., window..., heavy...]`` concatenated WITHOUT de-duplication and
    ``sparse_len`` filled with the row length.  With ``sorted_by_score`` the heavy part is
    in descending-score order like `torch.topk`; ties and the unsorted mode use the
    lowest-index rule."""
    B, H, L, R = q_probs.shape
    T = k_hard_bhlt.shape[-1]
    M_eff = min(M, T)
    scores = None
    heavy = np.empty((B, H, M_eff), dtype=np.int32)
    if M_eff > 0:
        scores = soft_hash_collision(q_probs, k_hard_bhlt.to(torch.int16), allowed_bht,
                                     v_norm_bht.float())
        s = scores.numpy()
        for b in range(B):
            for h in range(H):
                idx = topk_lowest_index(s[b, h], M_eff)
                if sorted_by_score:
                    idx = idx[np.lexsort((idx, -s[b, h, idx].astype(np.float64)))]
                heavy[b, h] = idx
    al = allowed_bht.numpy()
    if M_eff > 0:
        ok = np.take_along_axis(al, heavy.astype(np.int64), axis=-1)
        heavy = np.where(ok, heavy, -1).astype(np.int32)
    base = base_indices(T, sink, window)
    base = np.broadcast_to(base[None, None, :], (B, H, base.shape[0])).copy()
    base_ok = np.take_along_axis(al, base.astype(np.int64), axis=-1)
    base = np.where(base_ok, base, -1).astype(np.int32)
    sparse_list = np.concatenate([base, heavy], axis=-1)
    sparse_len = np.full((B, H), sparse_list.shape[-1], dtype=np.int32)
    return torch.from_numpy(sparse_list), torch.from_numpy(sparse_len), scores


# --------------------------------------------------------------------------------------
# sparse attention
# --------------------------------------------------------------------------------------
def sparse_attention_fwd(query, key, value, sparse_list, sparse_len, block_seq: int = 256,
                         skip_negative: bool = True) -> torch.Tensor:
    """out[b,h,:] = sum_j softmax_j(q.K[idx_j]/sqrt(D)) V[idx_j], j < sparse_len[b,h],
    repeated indices counted as often as they appear, KV head = h // rep.

    Restates the two-stage evaluation of GPT-FAST/kernels/sparse.py:102-235 in fp32: the
    list is cut into chunks of ``block_seq`` entries, each chunk is reduced with an online
    softmax over blocks of 16 entries (stage 1, :148-175, normalised partial and
    log-sum-exp stored :188-189), and the chunk partials are merged by their log-sum-exp
    (stage 2, :217-232).  ``skip_negative``: an index of -1 (masked entry) contributes
    nothing; the reference would read row -1 there, which never happens in decode because
    every position is allowed."""
    B, H, D = query.shape
    Hkv = key.shape[1]
    rep = H // Hkv
    scale = np.float32(1.0 / math.sqrt(D))
    q = query.float().numpy()
    k = key.float().numpy()
    v = value.float().numpy()
    lst = sparse_list.numpy()
    lens = sparse_len.numpy()
    out = np.zeros((B, H, D), dtype=np.float32)
    BLOCK_N = 16
    for b in range(B):
        for h in range(H):
            n = int(lens[b, h])
            kvh = h // rep
            part_o, part_lse = [], []
            for c0 in range(0, n, block_seq):
                c1 = min(n, c0 + block_seq)
                m = np.float32(-np.inf)
                se = np.float32(0.0)
                acc = np.zeros(D, dtype=np.float32)
                for s0 in range(c0, c1, BLOCK_N):
                    idx = lst[b, h, s0:min(c1, s0 + BLOCK_N)]
                    if skip_negative:
                        idx = idx[idx >= 0]
                        if idx.size == 0:
                            continue
                    kk = k[b, kvh, idx]
                    vv = v[b, kvh, idx]
                    att = (kk * q[b, h][None, :]).sum(axis=1, dtype=np.float32) * scale
                    new_m = np.maximum(att.max(), m)
                    p = np.exp(att - new_m, dtype=np.float32)
                    resc = np.exp(m - new_m, dtype=np.float32)
                    acc = acc * resc + (p[:, None] * vv).sum(axis=0, dtype=np.float32)
                    se = se * resc + p.sum(dtype=np.float32)
                    m = new_m
                if se > 0:
                    part_o.append(acc / se)
                    part_lse.append(m + np.log(se, dtype=np.float32))
            m = np.float32(-np.inf)
            se = np.float32(0.0)
            acc = np.zeros(D, dtype=np.float32)
            for o_c, lse_c in zip(part_o, part_lse):
                new_m = np.maximum(lse_c, m)
                old = np.exp(m - new_m, dtype=np.float32)
                w = np.exp(lse_c - new_m, dtype=np.float32)
                acc = acc * old + w * o_c
                se = se * old + w
                m = new_m
            out[b, h] = acc / se if se > 0 else 0.0
    return torch.from_numpy(out).to(query.dtype)


def sparse_attention_dense_check(query, key, value, sparse_list, sparse_len) -> torch.Tensor:
    """Same quantity by one fp64 gather + softmax per row (no chunking): an independent
    check of `sparse_attention_fwd` and of the kernels at sizes where the chunked loop is
    too slow."""
    B, H, D = query.shape
    rep = H // key.shape[1]
    out = torch.zeros(B, H, D, dtype=torch.float64)
    for b in range(B):
        for h in range(H):
            idx = sparse_list[b, h, : int(sparse_len[b, h])].long()
            idx = idx[idx >= 0]
            if idx.numel() == 0:
                continue
            kk = key[b, h // rep, idx].double()
            vv = value[b, h // rep, idx].double()
            s = (kk @ query[b, h].double()) / math.sqrt(D)
            out[b, h] = torch.softmax(s, dim=0) @ vv
    return out


# --------------------------------------------------------------------------------------
# whole decode step of one layer (what `Attention.sparse_forward` does between the QKV
# projection and the output projection, GPT-FAST/model.py:449-552)
# --------------------------------------------------------------------------------------
def decode_step(q_bhd, k_cache, v_cache, codes_bhtl, v_norm_bht, planes, protos_T,
                sink: int, window: int, M: int, temperature: float = 1.0):
    """Chained oracle on a cache that already contains the newly appended token.
    k_cache/v_cache [B,Hkv,T,D], codes [B,Hkv,T,L], v_norm [B,Hkv,T] fp16.
    Returns dict(q_probs, scores, sparse_list, sparse_len, out)."""
    B, H, D = q_bhd.shape
    Hkv = k_cache.shape[1]
    rep = H // Hkv
    T = k_cache.shape[2]
    q_probs = soft_hash(q_bhd, planes, protos_T, temperature)
    kh, vn = relayout_for_reference(codes_bhtl.to(torch.int16), v_norm_bht, rep)
    allowed = torch.ones(B, H, T, dtype=torch.bool)
    sparse_list, sparse_len, scores = build_sparse_list_decode(
        q_probs, kh, vn, allowed, sink, window, M)
    out = sparse_attention_fwd(q_bhd, k_cache, v_cache, sparse_list, sparse_len)
    return dict(q_probs=q_probs, scores=scores, sparse_list=sparse_list,
                sparse_len=sparse_len, out=out)
