"""The transformer harness on a GPU (`socket_b200/model.py`): the sparse decode step inside a
model, captured per token in a CUDA graph, against eager execution and against the CPU oracle."""
import pytest
import torch

from oracle import socket_oracle as orc
from socket_b200 import ops
from socket_b200.model import ModelArgs, Transformer, apply_rotary_emb, generate, precompute_freqs_cis

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _model(n_layer=2, **over):
    cfg = ModelArgs.from_name("tiny", n_layer=n_layer, **over)
    return Transformer(cfg).to(device=DEV, dtype=torch.bfloat16).init_random(seed=3, std=0.05)


@pytest.mark.parametrize("mode", ["sparse", "dense"])
def test_graph_replayed_decode_equals_eager_decode(mode):
    model = _model()
    prompt = torch.randint(0, model.config.vocab_size, (2, 700), generator=torch.Generator().manual_seed(0))
    a, st = generate(model, prompt, 12, mode=mode, use_graph=True)
    model.max_seq_length = -1
    b, _ = generate(model, prompt, 12, mode=mode, use_graph=False)
    assert torch.equal(a, b)
    assert st["decode_only_tokens"] == 2 * 11 and st["decode_time_s"] > 0
    assert (a[:, 700:] >= 0).all() and (a[:, 700:] < model.config.vocab_size).all()
    if mode == "sparse":
        assert all(int(l.attention.kv_cache.status) == 0 for l in model.layers)
        assert all(int(l.attention.kv_cache.prefill_len) == 700 + 11 for l in model.layers)


def test_sparse_layer_inside_the_model_matches_the_oracle():
    """One decode token, eagerly: the attention output of every layer, computed by the fused step
    from that layer's roped q / k / v and its cache, against the CPU oracle on the same cache."""
    model = _model(n_layer=2, heavy_const=96, sink_size=8, window_size=24)
    B, T = 2, 1500
    prompt = torch.randint(0, model.config.vocab_size, (B, T), generator=torch.Generator().manual_seed(1))
    model.setup_caches(B, T + 16)
    model.setup_decode(B, "sparse", use_graph=False)
    logits = model.prefill(prompt.to(DEV), chunk=512)
    model.start_decode(torch.argmax(logits, dim=-1, keepdim=True), T)
    model.decode_one_token()
    torch.cuda.synchronize()
    for layer in model.layers:
        a = layer.attention
        c = a.kv_cache
        assert int(c.status) == 0 and int(c.prefill_len) == T + 1
        k = c.k_cache[:, :, :T + 1].float().cpu()
        v = c.v_cache[:, :, :T + 1].float().cpu()
        codes = c.k_hard[:, :, :T + 1].cpu()
        exact, _ = orc.hard_hash_keys_exact(k.permute(0, 2, 1, 3), a.planes.float().cpu())
        assert torch.equal(codes.to(torch.int16), exact.permute(0, 2, 1, 3))
        res = orc.decode_step(a.q_s.float().cpu(), k, v, codes, c.v_norm[:, :, :T + 1].cpu(),
                              a.planes.float().cpu(), a.protos_T.cpu(), a.sink_size, a.window_size, a.heavy_const)
        assert (a.o_s.float().cpu() - res["out"].float()).abs().max() <= 2e-2
        # the newest token's K / V are the roped projections staged for the step
        assert torch.equal(c.k_cache[:, :, T], a.k_s[:, 0]) and torch.equal(c.v_cache[:, :, T], a.v_s[:, 0])


def test_sparse_decode_tracks_dense_decode_when_the_budget_covers_the_context():
    """With sink + window covering the whole (short) context and no top-k budget the sparse list
    is the full context without duplicates, so sparse and dense decoding pick the same tokens."""
    model = _model(n_layer=2, heavy_const=0, sink_size=0, window_size=4096)
    prompt = torch.randint(0, model.config.vocab_size, (1, 300), generator=torch.Generator().manual_seed(2))
    a, _ = generate(model, prompt, 8, mode="sparse", use_graph=False)
    model.max_seq_length = -1
    b, _ = generate(model, prompt, 8, mode="dense", use_graph=False)
    assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_rope_split_equals_the_tensor_formulation(dtype):
    B, H, Hkv, D, n_pos = 3, 8, 2, 128, 500
    g = torch.Generator().manual_seed(0)
    qkv = torch.randn(B, 1, (H + 2 * Hkv) * D, generator=g).to(dtype).to(DEV)
    table = precompute_freqs_cis(n_pos, D, 500000.0, device=DEV)
    pos = torch.tensor([317], device=DEV)
    q = torch.empty(B, H, D, dtype=dtype, device=DEV)
    k = torch.empty(B, 1, Hkv, D, dtype=dtype, device=DEV)
    v = torch.empty_like(k)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.rope_split(qkv, table, pos, H, Hkv, q, k, v, status=status)
    qq, kk, vv = qkv.split([H * D, Hkv * D, Hkv * D], dim=-1)
    want_q = apply_rotary_emb(qq.view(B, 1, H, D), table[pos])
    want_k = apply_rotary_emb(kk.view(B, 1, Hkv, D), table[pos])
    assert torch.equal(q, want_q.view(B, H, D)) and torch.equal(k, want_k) and torch.equal(v, vv.view(B, 1, Hkv, D))
    assert int(status) == 0
    # a position outside the table is reported, not read
    q.zero_()
    ops.rope_split(qkv, table, torch.tensor([n_pos], device=DEV), H, Hkv, q, k, v, status=status)
    torch.cuda.synchronize()
    assert int(status) == 1 and (q == 0).all()
