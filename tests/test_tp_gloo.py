"""World-size-2 CPU (gloo) check of the KV-head sharding logic in `socket_b200/tp.py`: every rank
runs the decode path on its own KV heads only (the CPU oracle stands in for the kernels, which need
a GPU), the per-rank outputs are gathered along the head axis, and the result must equal the
unsharded run bit for bit — heads are independent, so sharding may not change a single value."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import socket_oracle as orc
from socket_b200 import tp
from socket_b200.config import PRESETS
from socket_b200.synth import make_decode_inputs

B, H, HKV, T, M, SINK, WINDOW = 2, 8, 4, 640, 48, 4, 12


def _run_shard(inp, q, k, v):
    kh = orc.hard_hash_keys(k.permute(0, 2, 1, 3), inp.planes).permute(0, 2, 1, 3).to(torch.uint8)
    vn = orc.value_norm(v.permute(0, 2, 1, 3)).permute(0, 2, 1)
    return orc.decode_step(q, k, v, kh, vn, inp.planes, inp.protos_T, SINK, WINDOW, M)


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    assert tp.maybe_init_dist("gloo") == rank
    inp = make_decode_inputs(B, H, HKV, T, seed=77)
    q, k, v = tp.shard_heads(inp.q, inp.k, inp.v, world, rank)
    assert q.shape[1] == H // world and k.shape[1] == HKV // world
    res = _run_shard(inp, q.contiguous(), k.contiguous(), v.contiguous())
    full_out = tp.gather_heads(res["out"], world)
    full_list = tp.gather_heads(res["sparse_list"], world)
    y = torch.full((B, 1, 16), float(rank + 1))
    tp.all_reduce_sum(y)
    if rank == 0:
        ret["out"], ret["list"], ret["sum"] = full_out, full_list, y
    dist.barrier()
    dist.destroy_process_group()


def test_kv_head_sharding_reproduces_unsharded_result():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    inp = make_decode_inputs(B, H, HKV, T, seed=77)
    ref = _run_shard(inp, inp.q, inp.k, inp.v)
    assert torch.equal(ret["out"], ref["out"])
    assert torch.equal(ret["list"], ref["sparse_list"])
    assert (ret["sum"] == 3.0).all()


def test_head_ranges_follow_reference_partition():
    # tp.py:134-137 divides n_head and n_local_heads by the world size; rank r owns a contiguous block
    for world in (1, 2, 4, 8):
        seen_q, seen_kv = [], []
        for r in range(world):
            qs, ks = tp.head_ranges(32, 8, world, r)
            seen_q += list(range(32))[qs]
            seen_kv += list(range(8))[ks]
            assert (qs.stop - qs.start) // (ks.stop - ks.start) == 4      # GQA ratio preserved
            assert qs.start == ks.start * 4                               # query heads of those KV heads
        assert seen_q == list(range(32)) and seen_kv == list(range(8))
    with pytest.raises(ValueError):
        tp.head_ranges(32, 8, 3, 0)
    cfg = PRESETS["c3"].shard_kv_heads(8)
    assert cfg.n_head == 4 and cfg.n_local_heads == 1 and cfg.rep == 4
