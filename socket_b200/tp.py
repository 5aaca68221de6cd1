"""KV-head sharding of the sparse-attention path across the GPUs of one node.

The reference shards attention by heads (GPT-FAST/tp.py:134-137,146-148: `n_head`, `dim` and
`n_local_heads` are divided by the world size; `wqkv` is column-sharded per q/k/v block,
:73-91,129).  Every (batch, KV head) group of the sparse path is independent end to end —
hashing, codes, scoring, selection and attention never mix heads — so a rank that owns a
contiguous block of KV heads (and the query heads that map to them) runs the whole path
locally and the path itself needs no collective.  The only communication is the sum of the
output-projection partial results, which the reference registers as a forward hook
(tp.py:139-140) that does not fire on its sparse path; `all_reduce_sum` below is the
explicit call a caller issues after `wo`.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist


def maybe_init_dist(backend: Optional[str] = None) -> Optional[int]:
    """Join the process group described by the torchrun environment (RANK, WORLD_SIZE,
    MASTER_ADDR, MASTER_PORT).  Returns the rank, or None when run as a single process —
    the behaviour of GPT-FAST/tp.py:36-51."""
    world = int(os.environ.get("WORLD_SIZE", os.environ.get("LOCAL_WORLD_SIZE", "1")))
    if world < 2:
        return None
    rank = int(os.environ.get("RANK", os.environ.get("LOCAL_RANK", "0")))
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    if not dist.is_initialized():
        dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return rank


def head_ranges(n_head: int, n_local_heads: int, world_size: int, rank: int) -> Tuple[slice, slice]:
    """(query-head slice, KV-head slice) owned by `rank`."""
    if n_local_heads % world_size != 0 or n_head % world_size != 0:
        raise ValueError(f"{n_local_heads} KV heads / {n_head} query heads do not split over "
                         f"{world_size} ranks")
    kv_per = n_local_heads // world_size
    q_per = n_head // world_size
    return slice(rank * q_per, (rank + 1) * q_per), slice(rank * kv_per, (rank + 1) * kv_per)


def shard_heads(q_bhd: torch.Tensor, k_bhtd: torch.Tensor, v_bhtd: torch.Tensor, world_size: int,
                rank: int):
    """Rank-local views of q [B,H,D] and K/V [B,Hkv,T,D]."""
    qs, ks = head_ranges(q_bhd.shape[1], k_bhtd.shape[1], world_size, rank)
    return q_bhd[:, qs], k_bhtd[:, ks], v_bhtd[:, ks]


def gather_heads(out_local: torch.Tensor, world_size: int, group=None) -> torch.Tensor:
    """Concatenate the per-rank outputs [B,H/world,D] along the head axis (used by tests and
    by callers that want the full attention output rather than the summed projection)."""
    parts = [torch.empty_like(out_local) for _ in range(world_size)]
    dist.all_gather(parts, out_local.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def all_reduce_sum(y: torch.Tensor, group=None) -> torch.Tensor:
    """Sum of the row-sharded output projection over the ranks, full [B,S,dim] tensor
    (the reference's hook reduces only `output[0]`, GPT-FAST/tp.py:140)."""
    dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
    return y
