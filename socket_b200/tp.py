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


# ------------------------------------------------------------------------------------------
# Weight sharding of a whole model, the split GPT-FAST/tp.py:110-156 applies in place
# ------------------------------------------------------------------------------------------
def _rows(w: torch.Tensor, world_size: int, rank: int) -> torch.Tensor:
    assert w.size(0) % world_size == 0
    return torch.tensor_split(w, world_size, dim=0)[rank]


def _cols(w: torch.Tensor, world_size: int, rank: int) -> torch.Tensor:
    assert w.size(1) % world_size == 0
    return torch.tensor_split(w, world_size, dim=1)[rank]


def shard_qkv(wqkv: torch.Tensor, splits, world_size: int, rank: int) -> torch.Tensor:
    """Column-parallel shard of the fused projection: q, k and v blocks are each split over the
    ranks and re-concatenated, so a rank keeps whole heads (GPT-FAST/tp.py:73-77,124-129)."""
    q, k, v = wqkv.split(list(splits), dim=0)
    return torch.cat([_rows(q, world_size, rank), _rows(k, world_size, rank), _rows(v, world_size, rank)], dim=0)


@torch.no_grad()
def shard_transformer(full, world_size: int, rank: int):
    """Rank `rank`'s shard of a single-device `socket_b200.model.Transformer`: `wqkv`, `w1`, `w3`
    column-parallel, `wo`, `w2` row-parallel (GPT-FAST/tp.py:110-137), embeddings, norms, the
    vocabulary projection and the hash parameters replicated.  The sharded model sums the partial
    results of `wo` and `w2` over the ranks itself (`all_reduce_sum`)."""
    from .model import Transformer
    cfg = full.config
    dev, dt = full.tok_embeddings.weight.device, full.tok_embeddings.weight.dtype
    part = Transformer(cfg, world=world_size, rank=rank).to(device=dev, dtype=dt)
    part.tok_embeddings.weight.copy_(full.tok_embeddings.weight)
    part.norm.weight.copy_(full.norm.weight)
    part.output.weight.copy_(full.output.weight)
    for src, dst in zip(full.layers, part.layers):
        a, b = src.attention, dst.attention
        b.wqkv.weight.copy_(shard_qkv(a.wqkv.weight, [a.local_dim, a.kv_size, a.kv_size], world_size, rank))
        b.wo.weight.copy_(_cols(a.wo.weight, world_size, rank))
        b.planes.copy_(a.planes)
        b.protos_T.copy_(a.protos_T)
        dst.feed_forward.w1.copy_(_rows(src.feed_forward.w1, world_size, rank))
        dst.feed_forward.w3.copy_(_rows(src.feed_forward.w3, world_size, rank))
        dst.feed_forward.w2.weight.copy_(_cols(src.feed_forward.w2.weight, world_size, rank))
        dst.attention_norm.weight.copy_(src.attention_norm.weight)
        dst.ffn_norm.weight.copy_(src.ffn_norm.weight)
    return part


# ------------------------------------------------------------------------------------------
# Row-parallel projection fused with the sum over the ranks (decode, <= 8 rows)
# ------------------------------------------------------------------------------------------
class FusedRowParallel:
    """`out = res + sum_r x_r @ W_r^T` in one kernel per rank (`sk_gemv_allreduce`): what
    `wo` / `w2` followed by `all_reduce_sum` compute, without the separate collective.  The ranks
    exchange their partial rows through peer-mapped buffers that torch's symmetric memory
    allocates and maps (plumbing only: the kernel does the stores, the flags and the waits).

    One object serves every projection of the same output width: all ranks must call it in the
    same order.  `max_batch` <= 8."""

    def __init__(self, n_out: int, max_batch: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        from ._lib import lib
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.n_out, self.max_batch, self.device = n_out, max_batch, device
        nbytes = int(lib().sk_gemv_allreduce_buffer_bytes(self.world, max_batch, n_out))
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.counters = torch.zeros((n_out + 31) // 32, dtype=torch.int32, device=device)   # one per CTA
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.peer_base = int(self.handle.buffer_ptrs_dev)      # device array of the ranks' buffer addresses
        torch.cuda.synchronize(device)
        dist.barrier(self.group)                               # every rank's flags read zero before anyone calls

    def __call__(self, x: torch.Tensor, weight: torch.Tensor, res: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [..., K] (<= max_batch rows), weight [n_out, K] (this rank's input-column shard),
        res / out [..., n_out]."""
        from ._lib import check, dtype_code, lib, ptr, stream_ptr
        K = x.shape[-1]
        B = x.numel() // K
        assert weight.shape == (self.n_out, K) and weight.stride(1) == 1 and weight.dtype == x.dtype
        x = x.contiguous()
        if out is None:
            out = torch.empty(*x.shape[:-1], self.n_out, dtype=x.dtype, device=x.device)
        assert out.is_contiguous() and (res is None or (res.is_contiguous() and res.shape == out.shape))
        check(lib().sk_gemv_allreduce(ptr(x), ptr(weight), weight.stride(0), ptr(res), ptr(out), dtype_code(x), B,
                                      self.n_out, K, self.peer_base, self.world, self.rank, self.max_batch,
                                      ptr(self.counters), ptr(self.status), stream_ptr(x.device)),
              "sk_gemv_allreduce")
        return out
