"""Seeded random shapes through the fused paths: every way of building the list must agree with
the plain two-step path, and the fused decode step with the chain of separate calls."""
import random

import pytest
import torch

from socket_b200 import ops
from socket_b200.attention import SocketAttention
from socket_b200.synth import hypercube_protos, make_decode_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _shapes(seed, n, t_choices):
    rnd = random.Random(seed)
    out = []
    for _ in range(n):
        Hkv = rnd.choice([1, 2, 4, 8])
        H = Hkv * rnd.choice([1, 2, 4, 8])
        B = rnd.choice([1, 1, 2, 3])
        T = rnd.choice([rnd.randint(*r) for r in t_choices])
        M = rnd.choice([1, 7, 64, rnd.randint(1, max(1, T // 12)), rnd.randint(1, T + 5)])
        out.append((B, H, Hkv, T, M, rnd.choice([0, 1, 4, 64]), rnd.choice([0, 1, 16, 128]),
                    T + rnd.choice([0, 0, 37, 1000]), rnd.choice([None, None, rnd.randint(1, T)])))
    return out


@pytest.mark.parametrize("B,H,Hkv,T,M,sink,window,Tcap,T_live",
                         _shapes(7, 16, [(50, 3000), (4096, 20000), (20000, 70000)]))
def test_every_list_path_agrees_with_two_step(B, H, Hkv, T, M, sink, window, Tcap, T_live):
    g = torch.Generator().manual_seed(T + M)
    q = torch.randn(B, H, 128, generator=g)
    planes = torch.randn(32, 8, 128, generator=g)
    codes = torch.randint(0, 256, (B, Hkv, Tcap, 32), generator=g, dtype=torch.uint8).to(DEV)
    vn = (torch.rand(B, Hkv, Tcap, generator=g) * 3 + 0.5).to(torch.float16).to(DEV)
    _, lut = ops.soft_hash(q.to(DEV), planes.to(DEV), hypercube_protos(8).to(DEV), 1.0, n_kv_heads=Hkv,
                           want_probs=False, want_lut=True)
    Te = T if T_live is None else T_live
    T_dev = None if T_live is None else torch.tensor(T_live, dtype=torch.int32, device=DEV)
    scores = ops.score(lut, codes, vn, H, Te)
    want, want_len = ops.select_list(scores, Te, M, sink, window)
    k = want.shape[-1]
    results = []
    if ops.score_select_applicable(B, H, Hkv, 32, 256, T, M):
        got, got_len, _ = ops.score_select_list(lut, codes, vn, H, T, M, sink, window, T_dev=T_dev)
        results.append((got, got_len))
    if ops.score_select_cluster_size(B, H, Hkv, 32, 256, T, M):
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        got, got_len = ops.score_select_cluster(lut, codes, vn, H, T, M, sink, window, T_dev=T_dev, status=status)
        assert int(status) == 0
        results.append((got, got_len))
    for got, got_len in results:
        assert torch.equal(got_len, want_len)
        assert torch.equal(torch.sort(got[:, :, :k], -1).values, torch.sort(want, -1).values)


@pytest.mark.parametrize("B,H,Hkv,T,M,sink,window,_cap,_live",
                         _shapes(11, 10, [(40, 3000), (4096, 12000), (20000, 40000)]))
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_step_agrees_with_separate_calls(B, H, Hkv, T, M, sink, window, _cap, _live, dtype):
    M = min(M, T)
    inp = make_decode_inputs(B, H, Hkv, T + 2, seed=T + M, dtype=dtype)
    k_bshd = inp.k.permute(0, 2, 1, 3).contiguous().to(DEV)
    v_bshd = inp.v.permute(0, 2, 1, 3).contiguous().to(DEV)
    q = inp.q.to(DEV)
    state = {}
    for path in ("step", "calls"):
        attn = SocketAttention(H, Hkv, 128, heavy_const=M, sink_size=sink, window_size=window,
                               planes=inp.planes, protos_T=inp.protos_T, dtype=dtype, device=DEV)
        cache = attn.setup_cache(B, T + 50, dtype=dtype)
        cache.append(torch.arange(T, device=DEV), k_bshd[:, :T].contiguous(), v_bshd[:, :T].contiguous(), attn.planes)
        outs = []
        for i in range(2):
            kn, vn = k_bshd[:, T + i:T + i + 1].contiguous(), v_bshd[:, T + i:T + i + 1].contiguous()
            pos = torch.tensor([T + i], device=DEV)
            if path == "step":
                outs.append(attn.sparse_decode(q, kn, vn, pos).clone())
            else:
                cache.append(pos, kn, vn, attn.planes)
                Tn = T + i + 1
                _, lut = ops.soft_hash(q, attn.planes, attn.protos_T, 1.0, n_kv_heads=Hkv, want_probs=False,
                                       want_lut=True)
                sc = ops.score(lut, cache.k_hard, cache.v_norm, H, Tn)
                lst, ln = ops.select_list(sc, Tn, M, sink, window)
                outs.append(ops.sparse_decode(q, cache.k_cache, cache.v_cache, lst, ln, T=Tn))
        state[path] = (outs, cache.k_hard[:, :, :T + 2].clone(), cache.v_norm[:, :, :T + 2].clone(),
                       int(cache.prefill_len))
    a, b = state["step"], state["calls"]
    assert torch.equal(a[1], b[1]) and torch.equal(a[2], b[2]) and a[3] == b[3] == T + 2
    # same keys, possibly in another order: the outputs differ by rounding only
    tol = {torch.float32: 2e-5, torch.bfloat16: 1.6e-2}[dtype]
    for x, y in zip(a[0], b[0]):
        assert (x.float() - y.float()).abs().max().item() <= tol
