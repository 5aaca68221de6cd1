"""Full-size runs of the benchmark configurations (32K and 128K context) checked through
size-independent properties, since the CPU oracle would take too long there:

  * scores           == an fp32 torch gather-and-sum of the same table and codes (1e-5 rel.)
  * codes            == an fp64 torch projection sign on a sample of rows (bit-exact)
  * selection        the multiset of selected score values equals torch.topk's values
                     bit for bit, indices are unique and in range, sink/window prefix exact
  * attention        == an fp32 torch gather + softmax over the same list (2e-2 max-abs, bf16)
  * duplicates       repeating the whole list leaves the output unchanged
"""
import math

import pytest
import torch

from socket_b200 import ops
from socket_b200.attention import SocketAttention
from socket_b200.config import PRESETS
from socket_b200.synth import make_decode_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _torch_attention(q, k_cache, v_cache, lst, rep):
    B, H, D = q.shape
    out = torch.empty(B, H, D, dtype=torch.float32, device=q.device)
    for b in range(B):
        for h in range(H):
            idx = lst[b, h].long()
            idx = idx[idx >= 0]
            kk = k_cache[b, h // rep, idx].float()
            vv = v_cache[b, h // rep, idx].float()
            s = (kk @ q[b, h].float()) / math.sqrt(D)
            out[b, h] = torch.softmax(s, dim=0) @ vv
    return out


@pytest.mark.parametrize("preset", ["c2", "c3"])
def test_full_size_decode_step_properties(preset):
    cfg = PRESETS[preset]
    B, H, Hkv, T, D = cfg.batch, cfg.n_head, cfg.n_local_heads, cfg.context, cfg.head_dim
    rep = H // Hkv
    inp = make_decode_inputs(B, H, Hkv, T, seed=4321, dtype=torch.bfloat16, device=DEV)
    attn = SocketAttention(H, Hkv, D, L=cfg.L, P=cfg.P, heavy_const=cfg.topk, sink_size=cfg.sink,
                           window_size=cfg.window, planes=inp.planes, protos_T=inp.protos_T,
                           dtype=torch.bfloat16, device=DEV)
    Tcap = T + 64
    cache = attn.setup_cache(B, Tcap)
    k_bshd = inp.k.permute(0, 2, 1, 3)
    v_bshd = inp.v.permute(0, 2, 1, 3)
    chunk = 8192
    for s0 in range(0, T - 1, chunk):
        s1 = min(T - 1, s0 + chunk)
        cache.append(torch.arange(s0, s1, device=DEV), k_bshd[:, s0:s1].contiguous(),
                     v_bshd[:, s0:s1].contiguous(), attn.planes)
    q = inp.q.contiguous()
    out = torch.empty_like(q)
    step = ops.DecodeStep(cache, q, k_bshd[:, T - 1:T].contiguous(), v_bshd[:, T - 1:T].contiguous(),
                          torch.tensor([T - 1], device=DEV), attn.planes, attn.protos_T, out,
                          topk=cfg.topk, sink=cfg.sink, window=cfg.window, T_max=Tcap, keep_list=True)
    step.run()
    torch.cuda.synchronize()
    assert int(step.status) == 0 and int(cache.prefill_len) == T
    assert torch.equal(cache.k_cache[:, :, :T], inp.k) and torch.equal(cache.v_cache[:, :, :T], inp.v)

    # codes on a sample of rows, fp64 sign
    g = torch.Generator(device=DEV).manual_seed(1)
    rows = torch.randint(0, T, (512,), generator=g, device=DEV)
    proj = torch.einsum("bhtd,lpd->bhtlp", inp.k[:, :, rows].double(), inp.planes.double())
    w = (1 << torch.arange(cfg.P - 1, -1, -1, device=DEV)).long()
    want_codes = ((proj >= 0).long() * w).sum(-1)
    assert torch.equal(cache.k_hard[:, :, rows].long(), want_codes)

    # scores
    probs, lut = ops.soft_hash(q, attn.planes, attn.protos_T, 1.0, n_kv_heads=Hkv, want_lut=True)
    scores = ops.score(lut, cache.k_hard, cache.v_norm, H, T)
    codes_l = cache.k_hard[:, :, :T].long()                                   # [B,Hkv,T,L]
    for b in range(B):
        for h in range(0, H, 5):
            pr = probs[b, h]                                                  # [L,R]
            gathered = torch.gather(pr, 1, codes_l[b, h // rep].t())          # [L,T]
            want = gathered.sum(0) * cache.v_norm[b, h // rep, :T].float()
            torch.testing.assert_close(scores[b, h], want, rtol=1e-5, atol=0)

    # selection (the fused step selected on the same scores)
    ktot = cfg.ktot
    lst = step.list[:, :, :ktot]
    assert (step.list_len == ktot).all()
    nb = ktot - cfg.topk
    base = torch.cat([torch.arange(cfg.sink, device=DEV), torch.arange(T - cfg.window, T, device=DEV)])
    assert (lst[:, :, :nb] == base.int()).all()
    heavy = lst[:, :, nb:].long()
    assert heavy.min() >= 0 and heavy.max() < T
    srt = torch.sort(heavy, dim=-1).values
    assert (srt[..., 1:] != srt[..., :-1]).all()
    mine = torch.sort(torch.gather(scores, 2, heavy), dim=-1, descending=True).values
    ref = torch.topk(scores, cfg.topk, dim=-1).values
    assert torch.equal(mine, ref)

    # attention
    want = _torch_attention(q, cache.k_cache, cache.v_cache, lst, rep)
    assert (out.float() - want).abs().max() <= 2e-2
    dbl = torch.cat([lst, lst], dim=-1).contiguous()
    out2 = ops.sparse_decode(q, cache.k_cache, cache.v_cache, dbl,
                             torch.full((B, H), 2 * ktot, dtype=torch.int32, device=DEV), T=T)
    assert (out2.float() - out.float()).abs().max() <= 1e-2
