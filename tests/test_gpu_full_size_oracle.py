"""Full-size decode steps checked against the pinned CPU oracle (`oracle/c`, the plain-C
restatement that `tests/test_oracle_golden.py` ties to fixtures produced by the reference itself),
at the shapes the benchmark measures: the 32K and 128K configurations, the per-rank shapes of the
128K configuration when its 8 KV heads are split over 2, 4 and 8 GPUs, and the per-rank attention
shape of the 70B-style configuration (8 query heads on 1 KV head, batch 8, 64K context).

Everything goes through the C ABI.  Bars (the ones the reference's operator contract gives):

  * bucket codes       every code of the cache, incl. the appended token, equals the sign of the
                       exact (fp64) projection - bit-exact
  * value norms        fp16, at most one ulp from the oracle's on a few rows
  * scores             every head, <= 1e-5 relative to the oracle's fp32 scores
  * selection          `sk_select_list` fed the ORACLE's scores returns the oracle's index set
                       bit for bit (ties to the lowest index)
  * the fused step     its list equals the oracle's outside rounding-level near-ties of the k-th
                       score (2e-5 relative), prefix (sink, window) exact
  * attention output   <= 2e-2 max-abs against the oracle's attention over the step's own list
"""
import numpy as np
import pytest
import torch

from oracle import c_oracle
from socket_b200 import ops
from socket_b200.attention import SocketAttention
from socket_b200.synth import make_decode_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# (name, B, H, Hkv, T, top-k, sink, window)
SHAPES = [
    ("c2", 1, 32, 8, 32768, 1024, 64, 128),
    ("c3", 4, 32, 8, 131072, 2048, 64, 256),
    ("c3_rank_of_2", 4, 16, 4, 131072, 2048, 64, 256),
    ("c3_rank_of_4", 4, 8, 2, 131072, 2048, 64, 256),
    ("c3_rank_of_8", 4, 4, 1, 131072, 2048, 64, 256),
    ("c5_rank_of_8", 8, 8, 1, 65536, 2048, 64, 256),
]


@pytest.mark.parametrize("name,B,H,Hkv,T,M,sink,window", SHAPES, ids=[s[0] for s in SHAPES])
def test_full_size_step_against_the_cpu_oracle(name, B, H, Hkv, T, M, sink, window):
    D, L, P = 128, 32, 8
    dt = torch.bfloat16
    inp = make_decode_inputs(B, H, Hkv, T, seed=977, dtype=dt, device=DEV)
    attn = SocketAttention(H, Hkv, D, L=L, P=P, heavy_const=M, sink_size=sink, window_size=window,
                           planes=inp.planes, protos_T=inp.protos_T, dtype=dt, device=DEV)
    Tcap = T + 64
    cache = attn.setup_cache(B, Tcap)
    k_bshd = inp.k.permute(0, 2, 1, 3)
    v_bshd = inp.v.permute(0, 2, 1, 3)
    for s0 in range(0, T - 1, 8192):                       # prefill: the bulk (tensor-core) append
        s1 = min(T - 1, s0 + 8192)
        cache.append(torch.arange(s0, s1, device=DEV), k_bshd[:, s0:s1].contiguous(),
                     v_bshd[:, s0:s1].contiguous(), attn.planes)
    q = inp.q.contiguous()
    out = torch.empty_like(q)
    step = ops.DecodeStep(cache, q, k_bshd[:, T - 1:T].contiguous(), v_bshd[:, T - 1:T].contiguous(),
                          torch.tensor([T - 1], device=DEV), attn.planes, attn.protos_T, out,
                          topk=M, sink=sink, window=window, T_max=Tcap, keep_list=True)
    step.run()
    torch.cuda.synchronize()
    assert int(step.status) == 0 and int(cache.prefill_len) == T
    assert step.rescored_rows() in (None, 0)

    # ---- host copies, oracle side
    k_h, v_h, q_h = inp.k.cpu(), inp.v.cpu(), inp.q.cpu()
    planes_h, protos_h = inp.planes.cpu(), inp.protos_T.cpu()
    codes_gpu = cache.k_hard[:, :, :T].cpu()
    vn_gpu = cache.v_norm[:, :, :T].cpu()

    # bucket codes: every key of the cache (bulk path) and the appended token (decode path)
    exact = c_oracle.hash_keys(k_h, planes_h, exact=True)             # [B,Hkv,T,L] int16
    assert torch.equal(codes_gpu.to(torch.int16), exact), "bucket codes differ from the exact projection signs"
    del exact

    # value norms: fp32 norm rounded to fp16; the GPU sums in fp64 first
    vn_orc = c_oracle.value_norm(v_h)
    dv = (vn_gpu.view(torch.int16).int() - vn_orc.view(torch.int16).int()).abs()
    assert int(dv.max()) <= 1 and float((dv > 0).float().mean()) < 0.02

    # scores of every head
    qp = c_oracle.soft_hash(q_h, planes_h, protos_h)
    want_scores = c_oracle.score(qp, codes_gpu.contiguous(), vn_gpu.contiguous(), T)
    _, lut = ops.soft_hash(q, attn.planes, attn.protos_T, 1.0, n_kv_heads=Hkv, want_probs=False, want_lut=True)
    got_scores = ops.score(lut, cache.k_hard, cache.v_norm, H, T)
    torch.testing.assert_close(got_scores.cpu(), want_scores, rtol=1e-5, atol=0)
    del got_scores

    # the select kernel fed the oracle's scores
    want_list, want_len = c_oracle.select_list(want_scores, sink, window, M)
    ktot = want_list.shape[-1]
    got_list, got_len = ops.select_list(want_scores.to(DEV), T, M, sink, window)
    assert torch.equal(got_len.cpu(), want_len)
    nb = ktot - M
    assert torch.equal(got_list.cpu()[:, :, :nb], want_list[:, :, :nb])
    assert torch.equal(torch.sort(got_list.cpu()[:, :, nb:], dim=-1).values,
                       torch.sort(want_list[:, :, nb:], dim=-1).values)

    # the fused step's own list
    lst = step.list.cpu()[:, :, :ktot]
    assert (step.list_len.cpu() == ktot).all()
    assert torch.equal(lst[:, :, :nb], want_list[:, :, :nb])
    s = want_scores.numpy()
    for b in range(B):
        for h in range(H):
            got = np.sort(lst[b, h, nb:].numpy())
            want = np.sort(want_list[b, h, nb:].numpy())
            assert got.min() >= 0 and got.max() < T and (np.diff(got) > 0).all()
            if not np.array_equal(got, want):
                diff = np.setxor1d(got, want)
                kth = np.partition(s[b, h], T - M)[T - M]
                assert (np.abs(s[b, h][diff] - kth) <= 2e-5 * abs(kth)).all(), (name, b, h, len(diff))

    # attention over the step's own list
    want_out = c_oracle.sparse_attention(q_h, k_h, v_h, lst.contiguous(), step.list_len.cpu())
    assert (out.float().cpu() - want_out).abs().max() <= 2e-2
