"""Host-side checks of the transformer harness around the decode step (`socket_b200/model.py`)
that need no GPU: the rotary embedding, the dense reference flow on CPU (chunked causal prefill ==
one-shot prefill, decode continues it), and - as two gloo ranks - that the tensor-parallel shards
of `socket_b200/tp.py::shard_transformer` with their explicit all-reduces reproduce the
single-process model."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from socket_b200 import tp
from socket_b200.model import (ModelArgs, Transformer, apply_rotary_emb, generate, precompute_freqs_cis)


def _tiny(seed=0):
    torch.manual_seed(seed)
    cfg = ModelArgs.from_name("tiny", n_layer=2)
    return Transformer(cfg).float().init_random(seed=seed, std=0.05)


def test_rotary_matches_complex_rotation():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 5, 3, 16, generator=g)
    fc = precompute_freqs_cis(64, 16, base=10000.0).float()[7:12]
    got = apply_rotary_emb(x, fc)
    xc = torch.view_as_complex(x.reshape(2, 5, 3, 8, 2).contiguous())
    rot = torch.view_as_complex(fc.contiguous())[None, :, None, :]
    want = torch.view_as_real(xc * rot).flatten(3)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
    out = torch.empty(2, 5, 3, 16)
    apply_rotary_emb(x, fc, out=out)
    assert torch.equal(out, got)


def test_dense_flow_on_cpu_chunked_prefill_and_decode():
    model = _tiny()
    B, T, new = 2, 40, 6
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, model.config.vocab_size, (B, T + new), generator=g)
    model.setup_caches(B, T + new + 8)
    one = model.prefill(prompt[:, :T], chunk=4096)
    model.max_seq_length = -1
    model.setup_caches(B, T + new + 8)                      # fresh caches
    chunked = model.prefill(prompt[:, :T], chunk=16)
    torch.testing.assert_close(chunked, one, rtol=1e-4, atol=1e-4)
    # teacher-forced decode over the next tokens == prefill over the longer prompt
    model.setup_decode(B, "dense", use_graph=False)
    model.start_decode(prompt[:, T:T + 1], T)
    x = None
    for i in range(new):
        model._tok.copy_(prompt[:, T + i:T + i + 1])
        tok = model.decode_one_token()
    model.max_seq_length = -1
    model.setup_caches(B, T + new + 8)
    full = model.prefill(prompt[:, :T + new], chunk=4096)
    assert torch.equal(tok[:, 0], torch.argmax(full, dim=-1))


def test_generate_is_deterministic_on_cpu():
    model = _tiny(3)
    prompt = torch.randint(0, model.config.vocab_size, (1, 24), generator=torch.Generator().manual_seed(2))
    a, st = generate(model, prompt, 5, mode="dense", use_graph=False)
    model.max_seq_length = -1
    b, _ = generate(model, prompt, 5, mode="dense", use_graph=False)
    assert torch.equal(a, b) and a.shape == (1, 29) and st["decode_only_tokens"] == 4


def _tp_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    assert tp.maybe_init_dist("gloo") == rank
    full = _tiny(5)
    part = tp.shard_transformer(full, world, rank)
    a = part.layers[0].attention
    assert a.n_head == full.config.n_head // world and a.n_local_heads == full.config.n_local_heads // world
    assert a.wqkv.weight.shape[0] == (full.config.n_head + 2 * full.config.n_local_heads) // world * full.config.head_dim
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, full.config.vocab_size, (2, 20), generator=g)
    seq, _ = generate(part, prompt, 4, mode="dense", use_graph=False)
    part.max_seq_length = -1
    part.setup_caches(2, 32)
    logits = part.prefill(prompt)
    if rank == 0:
        ret["seq"], ret["logits"] = seq, logits
    dist.barrier()
    dist.destroy_process_group()


def test_tensor_parallel_shards_reproduce_the_single_process_model():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_tp_worker, args=(2, port, ret), nprocs=2, join=True)
    full = _tiny(5)
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, full.config.vocab_size, (2, 20), generator=g)
    seq, _ = generate(full, prompt, 4, mode="dense", use_graph=False)
    full.max_seq_length = -1
    full.setup_caches(2, 32)
    logits = full.prefill(prompt)
    torch.testing.assert_close(ret["logits"], logits, rtol=1e-4, atol=1e-4)
    assert torch.equal(ret["seq"], seq)
