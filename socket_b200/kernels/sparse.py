"""Drop-in replacement of `GPT-FAST/kernels/sparse.py`: the two operators
`Attention.sparse_forward` imports (GPT-FAST/model.py:16) with the same names, argument
order, dtypes, shapes and error behaviour, running on the hand-written sm_100a kernels.

    from socket_b200.kernels.sparse import build_sparse_list_decode, sparse_attention_fwd

Differences a caller can observe:
  * no host synchronisation inside either call (the reference syncs at sparse.py:64 and :320);
  * among equal scores the top-k keeps the smallest indices (`torch.topk` leaves the choice
    open); the top-k part is still ordered by descending score;
  * `sparse_attention_fwd` skips entries equal to -1 instead of reading row -1, and reads
    K/V in place, so the caller need not make the `[:, :, :T]` prefix contiguous
    (GPT-FAST/model.py:541-542).
"""
from __future__ import annotations

import torch

from .. import ops


@torch.no_grad()
def build_sparse_list_decode(
    q_probs: torch.Tensor,         # [B,H,L,R] fp16/bf16/fp32
    k_hard_bhlt: torch.Tensor,     # [B,H,L,T] int16/int32
    v_norm_bht: torch.Tensor,      # [B,H,T] fp16/bf16
    allowed_bht: torch.Tensor,     # [B,H,T] bool
    sink: int,
    window: int,
    M: int,
    KC: int = 8,
    BLOCK_N: int = 512,
    num_warps: int = 8,
    num_stages: int = 2,
):
    """Same contract as GPT-FAST/kernels/sparse.py:15-95.  Returns
    (sparse_list int32 [B,H,Ktot], sparse_len int32 [B,H]); the tuning arguments are accepted
    and ignored, as in the reference (:38)."""
    assert q_probs.is_cuda and k_hard_bhlt.is_cuda and v_norm_bht.is_cuda and allowed_bht.is_cuda
    assert q_probs.dtype in (torch.float16, torch.bfloat16, torch.float32)
    assert allowed_bht.dtype == torch.bool
    B, H, L, R = q_probs.shape
    _, _, L2, T = k_hard_bhlt.shape
    assert L2 == L
    M_eff = min(M, T)
    if M_eff > 0:
        key_buckets = k_hard_bhlt if k_hard_bhlt.dtype == torch.int16 else k_hard_bhlt.to(torch.int16)
        scores = ops.soft_hash_collision(
            q_probs.float().unsqueeze(2).contiguous(), key_buckets.contiguous(),
            allowed_bht.unsqueeze(2).contiguous(), v_norm_bht.float().unsqueeze(2).contiguous(),
        ).squeeze(2)
    else:
        scores = torch.empty(B, H, T, dtype=torch.float32, device=q_probs.device)
    return ops.select_list(scores, T, M_eff, sink, window, sorted_by_score=True, allowed=allowed_bht)


@torch.no_grad()
def build_sparse_list_native(
    q_probs: torch.Tensor,        # [B,H,L,R]
    codes_bhtl: torch.Tensor,     # [B,Hkv,Tcap,L] uint8, the cache's own layout
    v_norm_bht: torch.Tensor,     # [B,Hkv,Tcap] fp16
    T: int,
    sink: int,
    window: int,
    M: int,
    allowed_bht: torch.Tensor = None,
    sorted_by_score: bool = False,
    return_scores: bool = False,
):
    """The same list from the cache-native layout: no expansion of the codes to query heads
    and no transposition (the relayout of GPT-FAST/model.py:494-506 is not needed)."""
    assert q_probs.is_cuda and codes_bhtl.is_cuda and v_norm_bht.is_cuda
    B, H, L, R = q_probs.shape
    Hkv = codes_bhtl.shape[1]
    lut = ops.lut_from_probs(q_probs, Hkv)
    scores = ops.score(lut, codes_bhtl, v_norm_bht, H, T, R=R, allowed=allowed_bht)
    lst, ln = ops.select_list(scores, T, min(M, T), sink, window, sorted_by_score=sorted_by_score,
                              allowed=allowed_bht)
    return (lst, ln, scores) if return_scores else (lst, ln)


@torch.no_grad()
def sparse_attention_fwd(
    query: torch.Tensor,       # [B,H,D]
    key: torch.Tensor,         # [B,Kv,S,D]
    value: torch.Tensor,       # [B,Kv,S,D]
    sparse_list: torch.Tensor, # [B,H,Ktotal]
    sparse_len: torch.Tensor,  # [B,H]
    block_seq: int = 256,
) -> torch.Tensor:
    """Same contract as GPT-FAST/kernels/sparse.py:309-329; `block_seq` is accepted for
    compatibility (the split of the list over CTAs is chosen from the device size)."""
    assert query.is_cuda and key.is_cuda and value.is_cuda and sparse_list.is_cuda and sparse_len.is_cuda
    if sparse_list.dtype != torch.int32:
        sparse_list = sparse_list.to(torch.int32)
    if sparse_len.dtype != torch.int32:
        sparse_len = sparse_len.to(torch.int32)
    return ops.sparse_decode(query, key, value, sparse_list, sparse_len, T=key.shape[2])
