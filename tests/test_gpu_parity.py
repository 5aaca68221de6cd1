"""Parity of the CUDA path (called through the C-ABI) with the golden fixtures produced by
the reference's own code and with the CPU oracle.  Needs a B200.

Tolerances (stated once, used below):
  bucket codes            bit-exact against the fp64-arbitrated oracle; against the reference's
                          fp32 codes everywhere except inside the oracle's ambiguity band
  scores                  <= 1e-5 relative (fp32)
  top-k indices           bit-exact as sets when the select kernel is fed the reference's scores
  attention output        <= 2e-2 max-abs for bf16, <= 1e-4 for fp32 inputs
"""
import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle import socket_oracle as orc
from socket_b200 import ops
from socket_b200._lib import SK_DEV_INDEX_OUT_OF_RANGE, SK_DEV_POS_OUT_OF_RANGE
from socket_b200.attention import KVCache, SocketAttention
from socket_b200.kernels.sparse import (build_sparse_list_decode, build_sparse_list_native,
                                        sparse_attention_fwd)
from socket_b200.synth import hypercube_protos, make_decode_inputs
from tests.golden_util import OPS_CASES, load_model_flow, load_ops_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCORE_RTOL = 1e-5
OUT_ATOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 2e-2}


def cu(t):
    return t.to(DEV)


# ---------------------------------------------------------------------------- hashing
@pytest.mark.parametrize("name", OPS_CASES)
def test_hash_codes_bit_exact(name):
    c = load_ops_case(name)
    keys = c.k.permute(0, 2, 1, 3).contiguous()                      # [B,T,Hkv,D]
    exact, amb = orc.hard_hash_keys_exact(keys.float(), c.planes.float())
    got = ops.hash_keys(cu(keys), cu(c.planes)).cpu()
    assert got.dtype == torch.uint8
    assert torch.equal(got.to(torch.int16), exact)
    ref = c.codes.permute(0, 2, 1, 3).to(torch.int16)                # reference, fp32 summation
    assert ((got.to(torch.int16) != ref) & ~amb.any(-1)).sum() == 0
    got16 = ops.hash_keys(cu(keys), cu(c.planes), code_dtype=torch.int16).cpu()
    assert torch.equal(got16, exact)


def test_hash_other_plane_counts_and_dims():
    g = torch.Generator().manual_seed(3)
    for D, P, dt in ((128, 5, torch.float32), (64, 8, torch.bfloat16), (128, 12, torch.float16)):
        keys = torch.randn(37, D, generator=g).to(dt)
        planes = torch.randn(16, P, D, generator=g).to(dt)
        exact, _ = orc.hard_hash_keys_exact(keys.float()[None, :, None, :], planes.float())
        got = ops.hash_keys(cu(keys), cu(planes), code_dtype=torch.int16 if P > 8 else torch.uint8).cpu()
        assert torch.equal(got.to(torch.int16), exact[0, :, 0])


@pytest.mark.parametrize("name", ["tiny_rep4_f32", "tiny_rep4_bf16", "batch2_rep4_f32"])
def test_kv_append_fills_cache_like_reference(name):
    c = load_ops_case(name)
    B, Hkv, T, D, L = c.B, c.Hkv, c.T, c.D, c.L
    cache = KVCache(B, T + 8, Hkv, D, L=L, R=1 << c.P, dtype=c.dtype, device=DEV)
    planes = cu(c.planes)
    k_bshd = cu(c.k.permute(0, 2, 1, 3).contiguous())
    v_bshd = cu(c.v.permute(0, 2, 1, 3).contiguous())
    # bulk (prefill-like) append of the first T-3 tokens, then three single-token appends
    cache.append(torch.arange(T - 3, device=DEV), k_bshd[:, :T - 3], v_bshd[:, :T - 3], planes)
    assert int(cache.prefill_len) == T - 3
    for t in range(T - 3, T):
        cache.append(torch.tensor([t], device=DEV), k_bshd[:, t:t + 1], v_bshd[:, t:t + 1], planes)
    assert int(cache.prefill_len) == T and int(cache.status) == 0
    assert torch.equal(cache.k_cache[:, :, :T].cpu(), c.k) and torch.equal(cache.v_cache[:, :, :T].cpu(), c.v)
    exact, amb = orc.hard_hash_keys_exact(c.k.float().permute(0, 2, 1, 3), c.planes.float())
    assert torch.equal(cache.k_hard[:, :, :T].cpu().to(torch.int16), exact.permute(0, 2, 1, 3))
    vn = cache.v_norm[:, :, :T].cpu()
    ulp = (vn.view(torch.int16).int() - c.v_norm.view(torch.int16).int()).abs()
    assert ulp.max() <= 1 and (ulp > 0).float().mean() < 0.02
    assert (cache.k_cache[:, :, T:] == 0).all() and (cache.k_hard[:, :, T:] == 0).all()
    # a position outside the cache is flagged and not written
    cache.append(torch.tensor([T + 8], device=DEV), k_bshd[:, :1], v_bshd[:, :1], planes)
    assert int(cache.status) & SK_DEV_POS_OUT_OF_RANGE
    assert int(cache.prefill_len) == T


def test_kvcache_update_contract():
    c = load_ops_case("tiny_rep4_f32")
    cache = KVCache(c.B, c.T, c.Hkv, c.D, L=c.L, R=256, dtype=torch.float32, device=DEV)
    k_bshd = cu(c.k.permute(0, 2, 1, 3))
    v_bshd = cu(c.v.permute(0, 2, 1, 3))
    attn = SocketAttention(c.H, c.Hkv, c.D, planes=c.planes, protos_T=c.protos_T, dtype=torch.float32,
                           device=DEV)
    k_hard = attn.hard_hash_keys(k_bshd)
    assert k_hard.dtype == torch.int16 and k_hard.shape == (c.B, c.T, c.Hkv, c.L)
    vn = torch.linalg.vector_norm(v_bshd.float(), ord=2, dim=-1).to(torch.float16)
    kc, vc = cache.update(torch.arange(c.T, device=DEV), k_bshd, v_bshd, v_norm=vn, k_hard=k_hard)
    assert kc is cache.k_cache and int(cache.prefill_len) == c.T
    assert torch.equal(cache.k_hard.cpu(), c.codes)
    with pytest.raises(RuntimeError, match="out-of-bounds"):
        cache.update(torch.tensor([c.T], device=DEV), k_bshd[:, :1], v_bshd[:, :1])
    bits = torch.tensor([[True, False, True, True, False, False, False, True]], device=DEV)
    assert attn.pack_bits(bits).item() == 0b10110001


# ---------------------------------------------------------------------------- soft hash
@pytest.mark.parametrize("name", ["tiny_rep4_f32", "tiny_rep4_bf16"])
def test_soft_hash_matches_reference(name):
    c = load_ops_case(name)
    probs, lut = ops.soft_hash(cu(c.q), cu(c.planes), cu(c.protos_T), 1.0, n_kv_heads=c.Hkv,
                               want_probs=True, want_lut=True)
    torch.testing.assert_close(probs.cpu(), c.q_probs, rtol=SCORE_RTOL, atol=1e-9)
    lut2 = ops.lut_from_probs(probs, c.Hkv)
    assert torch.equal(lut, lut2)
    ht = 4
    view = lut.view(c.B * c.Hkv, c.rep // ht, 256, c.L, ht).cpu()
    expect = c.q_probs.view(c.B * c.Hkv, c.rep // ht, ht, c.L, 256).permute(0, 1, 4, 3, 2)
    torch.testing.assert_close(view, expect, rtol=SCORE_RTOL, atol=1e-9)


def test_soft_hash_temperature_and_head_tiles():
    g = torch.Generator().manual_seed(9)
    for H, Hkv in ((2, 2), (4, 2), (8, 1), (3, 3)):
        q = torch.randn(2, H, 128, generator=g)
        planes = torch.randn(32, 8, 128, generator=g)
        protos = hypercube_protos(8)
        for temp in (1.0, 0.3):
            want = orc.soft_hash(q, planes, protos, temp)
            probs, lut = ops.soft_hash(cu(q), cu(planes), cu(protos), temp, n_kv_heads=Hkv, want_lut=True)
            torch.testing.assert_close(probs.cpu(), want, rtol=2e-5, atol=1e-9)
            assert torch.equal(lut, ops.lut_from_probs(probs, Hkv))


# ---------------------------------------------------------------------------- scorer
@pytest.mark.parametrize("name", OPS_CASES + ["c1_config"])
def test_scores_match_reference(name):
    c = load_ops_case(name)
    qp = c.q_probs if c.q_probs is not None else orc.soft_hash(c.q.float(), c.planes.float(), c.protos_T)
    codes = c.codes if c.codes is not None else \
        orc.hard_hash_keys(c.k.float().permute(0, 2, 1, 3), c.planes.float()).permute(0, 2, 1, 3).to(torch.uint8)
    vn = c.v_norm if c.v_norm is not None else orc.value_norm(c.v.float().permute(0, 2, 1, 3)).permute(0, 2, 1)
    want = c.scores if c.q_probs is not None else orc.score_keys_native(qp, codes, vn, c.allowed)
    lut = ops.lut_from_probs(cu(qp), c.Hkv)
    allowed = None if bool(c.allowed.all()) else cu(c.allowed)
    got = ops.score(lut, cu(codes.contiguous()), cu(vn.contiguous()), c.H, c.T, allowed=allowed).cpu()
    finite = torch.isfinite(want)
    assert torch.equal(torch.isfinite(got), finite)
    torch.testing.assert_close(got[finite], want[finite], rtol=SCORE_RTOL, atol=0)
    # the reference-surface entry point adds the tables in the reference's order: same bits
    kh, vn_h = orc.relayout_for_reference(codes.to(torch.int16), vn, c.rep)
    got2 = ops.soft_hash_collision(cu(qp.float().unsqueeze(2).contiguous()), cu(kh),
                                   cu(c.allowed.unsqueeze(2).contiguous()),
                                   cu(vn_h.float().unsqueeze(2).contiguous())).squeeze(2).cpu()
    assert torch.equal(got2, want)


def test_scores_on_a_cache_with_spare_capacity_and_device_length():
    c = load_ops_case("batch2_rep4_f32")
    Tcap = c.T + 100
    codes = torch.zeros(c.B, c.Hkv, Tcap, c.L, dtype=torch.uint8)
    codes[:, :, :c.T] = c.codes
    vn = torch.zeros(c.B, c.Hkv, Tcap, dtype=torch.float16)
    vn[:, :, :c.T] = c.v_norm
    qp = orc.soft_hash(c.q.float(), c.planes.float(), c.protos_T)
    lut = ops.lut_from_probs(cu(qp), c.Hkv)
    T_dev = torch.tensor(c.T, dtype=torch.int32, device=DEV)
    out = torch.full((c.B, c.H, Tcap), 123.0, device=DEV)
    ops.score(lut, cu(codes), cu(vn), c.H, Tcap, T_dev=T_dev, out=out)
    torch.testing.assert_close(out[:, :, :c.T].cpu(), c.scores, rtol=SCORE_RTOL, atol=0)
    assert (out[:, :, c.T:] == 123.0).all()          # nothing written past the live length


# ---------------------------------------------------------------------------- select + list
def _check_rows(scores, lst, ln, T, sink, window, M, allowed=None, sorted_by_score=False):
    B, H = scores.shape[:2]
    base = orc.base_indices(T, sink, window)
    nb = base.shape[0]
    k_eff = min(M, T)
    assert lst.shape[-1] == nb + k_eff and (ln == nb + k_eff).all()
    for b in range(B):
        for h in range(H):
            s = scores[b, h, :T]
            al = allowed[b, h] if allowed is not None else np.ones(T, dtype=bool)
            assert np.array_equal(lst[b, h, :nb], np.where(al[base], base, -1))
            want = orc.topk_lowest_index(s, k_eff)
            got = lst[b, h, nb:]
            want_masked = np.where(al[want], want, -1)
            if sorted_by_score:
                order = np.lexsort((want, -s[want].astype(np.float64)))
                assert np.array_equal(got, want_masked[order])
            else:
                    # deterministic but unspecified order: compare as sorted index sets
                    assert np.array_equal(np.sort(got), np.sort(want_masked))


@pytest.mark.parametrize("name", OPS_CASES + ["c1_config"])
@pytest.mark.parametrize("sorted_by_score", [False, True])
def test_select_fed_reference_scores_is_bit_exact(name, sorted_by_score):
    c = load_ops_case(name)
    allowed = None if bool(c.allowed.all()) else cu(c.allowed)
    lst, ln = ops.select_list(cu(c.scores), c.T, c.M, c.sink, c.window, sorted_by_score=sorted_by_score,
                              allowed=allowed)
    _check_rows(c.scores.numpy(), lst.cpu().numpy(), ln.cpu().numpy(), c.T, c.sink, c.window, c.M,
                None if allowed is None else c.allowed.numpy(), sorted_by_score)
    # the reference's own list holds the same index set wherever its cut is free of ties
    ref = c.sparse_list.numpy()
    got = lst.cpu().numpy()
    for b in range(c.B):
        for h in range(c.H):
            s = c.scores[b, h].numpy()
            kept = ref[b, h][ref[b, h] >= 0]
            if np.unique(s).shape[0] == s.shape[0]:
                assert sorted(got[b, h][got[b, h] >= 0].tolist()) == sorted(kept.tolist())


@pytest.mark.parametrize("T,M,kind", [
    (1, 1, "normal"), (17, 5, "normal"), (255, 255, "normal"), (256, 100, "ties"), (257, 300, "normal"),
    (4096, 256, "ties"), (16384, 1000, "normal"), (16385, 1000, "normal"), (40000, 2048, "normal"),
    (40000, 1024, "ties"), (40000, 3000, "equal"), (70000, 16, "inf"), (131072, 2048, "heavy"),
    (100000, 1, "normal"), (50000, 49999, "normal"), (33333, 4096, "twolevel"),
])
def test_select_stress(T, M, kind):
    g = torch.Generator().manual_seed(T * 7 + M)
    rows = 3
    if kind == "normal":
        s = torch.rand(1, rows, T, generator=g) * 3 + 0.01
    elif kind == "ties":
        s = torch.randint(0, 50, (1, rows, T), generator=g).float() * 0.125
    elif kind == "equal":
        s = torch.full((1, rows, T), 0.75)
    elif kind == "inf":
        s = torch.rand(1, rows, T, generator=g)
        s[:, :, ::3] = float("-inf")
        s[:, 1] = float("-inf")
        s[:, 1, 5] = 1.0
    elif kind == "heavy":
        s = torch.rand(1, rows, T, generator=g) * 0.3 + 0.5
        idx = torch.randperm(T, generator=g)[: T // 100]
        s[:, :, idx] *= 8.0
        s[:, 2] = torch.exp(torch.randn(T, generator=g) * 4)
    else:  # two populations, the cut falls inside a large group of equal values
        s = torch.rand(1, rows, T, generator=g)
        s[:, :, : T // 2] = 2.0
    for sorted_by_score in (False, True):
        if sorted_by_score and min(M, T) > 16384:
            continue
        lst, ln = ops.select_list(cu(s), T, M, 2, 3, sorted_by_score=sorted_by_score)
        _check_rows(s.numpy(), lst.cpu().numpy(), ln.cpu().numpy(), T, 2, 3, M,
                    sorted_by_score=sorted_by_score)


def test_select_with_device_length_and_row_stride():
    g = torch.Generator().manual_seed(1)
    T, Tmax = 5000, 6000
    s = torch.rand(2, 4, Tmax, generator=g)
    T_dev = torch.tensor(T, dtype=torch.int32, device=DEV)
    lst, ln = ops.select_list(cu(s), Tmax, 64, 4, 16, T_dev=T_dev)
    lst, ln = lst.cpu().numpy(), ln.cpu().numpy()
    k = orc.base_indices(T, 4, 16).shape[0] + 64
    assert (ln == k).all()
    _check_rows(s.numpy(), lst[:, :, :k], ln, T, 4, 16, 64)


# ---------------------------------------------------------------------------- sparse attention
@pytest.mark.parametrize("name", OPS_CASES + ["c1_config"])
def test_sparse_attention_matches_reference(name):
    c = load_ops_case(name)
    q, k, v = cu(c.q), cu(c.k), cu(c.v)
    out = sparse_attention_fwd(q, k, v, cu(c.sparse_list), cu(c.sparse_len))
    assert out.dtype == c.q.dtype and out.shape == c.q.shape
    if c.out is not None:
        want = c.out
    else:   # lists with -1 entries: the reference kernel is undefined there, the oracle skips them
        want = orc.sparse_attention_dense_check(c.q.float(), c.k.float(), c.v.float(), c.sparse_list,
                                                c.sparse_len).float()
    assert (out.float().cpu() - want).abs().max() <= OUT_ATOL[c.q.dtype]


def test_sparse_attention_in_place_cache_views_and_bad_indices():
    c = load_ops_case("tiny_rep4_bf16")
    Tcap = c.T + 56
    kc = torch.zeros(c.B, c.Hkv, Tcap, c.D, dtype=c.dtype, device=DEV)
    vc = torch.zeros_like(kc)
    kc[:, :, :c.T] = cu(c.k)
    vc[:, :, :c.T] = cu(c.v)
    a = sparse_attention_fwd(cu(c.q), kc[:, :, :c.T], vc[:, :, :c.T], cu(c.sparse_list), cu(c.sparse_len))
    b = sparse_attention_fwd(cu(c.q), cu(c.k), cu(c.v), cu(c.sparse_list), cu(c.sparse_len))
    assert torch.equal(a, b)
    # duplicated entries count twice: doubling the whole list leaves the output unchanged
    dbl = torch.cat([c.sparse_list, c.sparse_list], dim=-1)
    d = sparse_attention_fwd(cu(c.q), cu(c.k), cu(c.v), cu(dbl), cu(c.sparse_len * 2))
    assert (d.float() - b.float()).abs().max() <= 1e-2
    # an index past the live length is skipped and reported, not dereferenced
    bad = c.sparse_list.clone()
    bad[0, 0, 3] = c.T + 5
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    e = ops.sparse_decode(cu(c.q), cu(c.k), cu(c.v), cu(bad), cu(c.sparse_len), T=c.T, status=status)
    assert int(status) & SK_DEV_INDEX_OUT_OF_RANGE
    skip = c.sparse_list.clone()
    skip[0, 0, 3] = -1
    f = sparse_attention_fwd(cu(c.q), cu(c.k), cu(c.v), cu(skip), cu(c.sparse_len))
    assert torch.equal(e, f)
    # shorter per-row lengths
    ln = c.sparse_len.clone()
    ln[0, 1] = 7
    ln[0, 2] = 0
    gl = sparse_attention_fwd(cu(c.q), cu(c.k), cu(c.v), cu(c.sparse_list), cu(ln))
    want = orc.sparse_attention_dense_check(c.q.float(), c.k.float(), c.v.float(), c.sparse_list, ln).float()
    assert (gl.float().cpu() - want).abs().max() <= 2e-2
    assert (gl[0, 2] == 0).all()


# ---------------------------------------------------------------------------- drop-in operators
@pytest.mark.parametrize("name", OPS_CASES)
def test_build_sparse_list_decode_reference_surface(name):
    c = load_ops_case(name)
    qp = c.q_probs if c.q_probs is not None else orc.soft_hash(c.q.float(), c.planes.float(), c.protos_T)
    kh, vn = orc.relayout_for_reference(c.codes.to(torch.int16), c.v_norm, c.rep)
    lst, ln = build_sparse_list_decode(cu(qp), cu(kh), cu(vn), cu(c.allowed), sink=c.sink, window=c.window,
                                       M=c.M, KC=8, BLOCK_N=512, num_warps=8, num_stages=2)
    assert lst.dtype == torch.int32 and ln.dtype == torch.int32
    assert lst.shape == c.sparse_list.shape and torch.equal(ln.cpu(), c.sparse_len)
    _check_rows(c.scores.numpy(), lst.cpu().numpy(), ln.cpu().numpy(), c.T, c.sink, c.window, c.M,
                c.allowed.numpy(), sorted_by_score=True)
    # native layout gives the same sets
    allowed = None if bool(c.allowed.all()) else cu(c.allowed)
    lst2, ln2, sc2 = build_sparse_list_native(cu(qp), cu(c.codes), cu(c.v_norm), c.T, c.sink, c.window, c.M,
                                              allowed_bht=allowed, return_scores=True)
    fin = torch.isfinite(c.scores)
    torch.testing.assert_close(sc2.cpu()[fin], c.scores[fin], rtol=SCORE_RTOL, atol=0)


def test_model_flow_decode_step_matches_reference():
    """The reference's whole sparse_forward (prefill + one decode step) against the fused
    decode step running on a cache filled by the fused append."""
    m = load_model_flow()
    B, H, D = m.q.shape
    Hkv, Tcap, L = m.k_cache.shape[1], m.k_cache.shape[2], m.planes.shape[0]
    attn = SocketAttention(H, Hkv, D, L=L, P=8, heavy_const=m.M, sink_size=m.sink, window_size=m.window,
                           planes=m.planes, protos_T=m.protos_T, dtype=torch.float32, device=DEV)
    cache = attn.setup_cache(B, Tcap, dtype=torch.float32)
    S = m.S
    cache.append(torch.arange(S, device=DEV), cu(m.k_prefill), cu(m.v_cache[:, :, :S].permute(0, 2, 1, 3).contiguous()),
                 attn.planes)
    v_step = m.v_cache[:, :, S:S + 1].permute(0, 2, 1, 3).contiguous()
    out = attn.sparse_decode(cu(m.q), cu(m.k_step), cu(v_step), torch.tensor([S], device=DEV))
    assert int(cache.prefill_len) == m.T
    assert torch.equal(cache.k_hard[:, :, :m.T].cpu(), m.codes[:, :, :m.T])
    assert (out.cpu() - m.out_bhd).abs().max() <= OUT_ATOL[torch.float32]
    step = attn._step[1]
    assert int(step.status) == 0


def test_steps_across_a_partly_filled_chunk_never_rescore():
    """While the context grows through a scorer chunk, that chunk holds a handful of keys, then a few
    hundred: at every fill level its cut must stay below each row's k-th score and its runs must not
    overflow, or the row drops to the select kernel's rescoring path (exact, but many times slower)."""
    B, H, Hkv, M, sink, window = 1, 32, 8, 1024, 64, 128
    Tcap = 34872                                   # 18 chunks of 1952 slots per KV head; one starts at 33184
    T0, steps = 33150, 1150
    inp = make_decode_inputs(B, H, Hkv, T0, seed=1234, dtype=torch.bfloat16)
    attn = SocketAttention(H, Hkv, 128, heavy_const=M, sink_size=sink, window_size=window,
                           planes=inp.planes, protos_T=inp.protos_T, dtype=torch.bfloat16, device=DEV)
    cache = attn.setup_cache(B, Tcap, dtype=torch.bfloat16)
    k_bshd, v_bshd = inp.k.permute(0, 2, 1, 3), inp.v.permute(0, 2, 1, 3)
    for s0 in range(0, T0, 8192):
        s1 = min(T0, s0 + 8192)
        cache.append(torch.arange(s0, s1, device=DEV), cu(k_bshd[:, s0:s1].contiguous()),
                     cu(v_bshd[:, s0:s1].contiguous()), attn.planes)
    g = torch.Generator().manual_seed(77)
    q_all = cu(torch.randn(steps, B, H, 128, generator=g).to(torch.bfloat16))
    k_all = cu(torch.randn(steps, B, 1, Hkv, 128, generator=g).to(torch.bfloat16))
    v_all = cu(torch.randn(steps, B, 1, Hkv, 128, generator=g).to(torch.bfloat16))
    q = torch.empty(B, H, 128, dtype=torch.bfloat16, device=DEV)
    kn = torch.empty(B, 1, Hkv, 128, dtype=torch.bfloat16, device=DEV)
    vn = torch.empty_like(kn)
    pos = torch.zeros(1, dtype=torch.int64, device=DEV)
    out = torch.empty_like(q)
    step = ops.DecodeStep(cache, q, kn, vn, pos, attn.planes, attn.protos_T, out, topk=M, sink=sink,
                          window=window, T_max=Tcap)
    assert step.rescored_rows() == 0
    for i in range(steps):
        q.copy_(q_all[i]); kn.copy_(k_all[i]); vn.copy_(v_all[i]); pos.fill_(T0 + i)
        step.run()
    torch.cuda.synchronize()
    assert int(step.status) == 0 and int(cache.prefill_len) == T0 + steps
    assert step.rescored_rows() == 0
    assert torch.isfinite(out.float()).all()


def test_graph_replayed_steps_see_the_newest_token():
    """The step's kernels are chained so that each may start while its predecessor drains.  Replayed
    from a CUDA graph they do overlap, and every replay must still score and attend over the token
    its own first kernel appended: compare each replay with separate, unchained calls."""
    B, H, Hkv, T, M, sink, window = 2, 8, 2, 5000, 128, 8, 24
    inp = make_decode_inputs(B, H, Hkv, T + 4, seed=33, dtype=torch.bfloat16)
    k_bshd = cu(inp.k.permute(0, 2, 1, 3).contiguous())
    v_bshd = cu(inp.v.permute(0, 2, 1, 3).contiguous())
    attn = SocketAttention(H, Hkv, 128, heavy_const=M, sink_size=sink, window_size=window,
                           planes=inp.planes, protos_T=inp.protos_T, dtype=torch.bfloat16, device=DEV)
    cache = attn.setup_cache(B, T + 64, dtype=torch.bfloat16)
    cache.append(torch.arange(T, device=DEV), k_bshd[:, :T].contiguous(), v_bshd[:, :T].contiguous(), attn.planes)
    q = cu(inp.q)
    kn = torch.empty(B, 1, Hkv, 128, dtype=torch.bfloat16, device=DEV)
    vn = torch.empty_like(kn)
    pos = torch.zeros(1, dtype=torch.int64, device=DEV)
    out = torch.empty_like(q)
    step = ops.DecodeStep(cache, q, kn, vn, pos, attn.planes, attn.protos_T, out, topk=M, sink=sink,
                          window=window, T_max=T + 64, keep_list=True)
    kn.copy_(k_bshd[:, T:T + 1]); vn.copy_(v_bshd[:, T:T + 1]); pos.fill_(T)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        step.run()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step.run()
    for i in range(4):
        kn.copy_(k_bshd[:, T + i:T + i + 1]); vn.copy_(v_bshd[:, T + i:T + i + 1]); pos.fill_(T + i)
        q.copy_(cu(inp.q) * (1.0 + 0.25 * i))                      # a different table every replay
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        Tn = T + i + 1
        assert int(step.status) == 0 and int(cache.prefill_len) == Tn
        _, lut = ops.soft_hash(q, attn.planes, attn.protos_T, 1.0, n_kv_heads=Hkv, want_probs=False, want_lut=True)
        sc = ops.score(lut, cache.k_hard, cache.v_norm, H, Tn)
        lst, ln = ops.select_list(sc, Tn, M, sink, window)
        ref = ops.sparse_decode(q, cache.k_cache, cache.v_cache, lst, ln, T=Tn)
        ktot = lst.shape[-1]
        assert torch.equal(step.list_len, ln)
        assert torch.equal(torch.sort(step.list[:, :, :ktot], -1).values, torch.sort(lst, -1).values), i
        assert (lst == Tn - 1).any(dim=-1).all()                   # the window holds the newest token
        got = ops.sparse_decode(q, cache.k_cache, cache.v_cache, step.list[:, :, :ktot].contiguous(),
                                step.list_len, T=Tn)
        assert torch.equal(out, got), i


def test_host_decoder_equals_device_path():
    """The host-memory entry (pinned staging -> graph of copy, step, copy back) gives the same
    bits as the device-tensor call on the same cache, and advances the cache the same way."""
    B, H, Hkv, T, M, sink, window = 2, 8, 2, 5000, 128, 8, 24
    inp = make_decode_inputs(B, H, Hkv, T + 2, seed=33, dtype=torch.bfloat16)
    k_bshd = inp.k.permute(0, 2, 1, 3).contiguous()
    v_bshd = inp.v.permute(0, 2, 1, 3).contiguous()
    outs = []
    for mode in ("device", "host"):
        attn = SocketAttention(H, Hkv, 128, heavy_const=M, sink_size=sink, window_size=window,
                               planes=inp.planes, protos_T=inp.protos_T, dtype=torch.bfloat16, device=DEV)
        cache = attn.setup_cache(B, T + 64, dtype=torch.bfloat16)
        cache.append(torch.arange(T, device=DEV), cu(k_bshd[:, :T]), cu(v_bshd[:, :T]), attn.planes)
        got = []
        hd = attn.host_decoder(B) if mode == "host" else None
        for i in range(2):
            kn, vn = k_bshd[:, T + i:T + i + 1].contiguous(), v_bshd[:, T + i:T + i + 1].contiguous()
            if mode == "host":
                o = hd(inp.q, kn, vn, T + i).clone()
            else:
                o = attn.sparse_decode(cu(inp.q), cu(kn), cu(vn), torch.tensor([T + i], device=DEV)).cpu()
            got.append(o)
        assert int(cache.prefill_len) == T + 2
        outs.append((got, cache.k_hard[:, :, :T + 2].cpu(), cache.v_norm[:, :, :T + 2].cpu()))
    for a, b in zip(outs[0][0], outs[1][0]):
        assert torch.equal(a, b)
    assert torch.equal(outs[0][1], outs[1][1]) and torch.equal(outs[0][2], outs[1][2])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_decode_step_against_chained_oracle(dtype):
    B, H, Hkv, T, M, sink, window = 2, 8, 2, 3000, 96, 8, 24
    inp = make_decode_inputs(B, H, Hkv, T + 1, seed=21, dtype=dtype)
    attn = SocketAttention(H, Hkv, 128, heavy_const=M, sink_size=sink, window_size=window,
                           planes=inp.planes, protos_T=inp.protos_T, dtype=dtype, device=DEV)
    cache = attn.setup_cache(B, T + 64, dtype=dtype)
    k_bshd = cu(inp.k.permute(0, 2, 1, 3).contiguous())
    v_bshd = cu(inp.v.permute(0, 2, 1, 3).contiguous())
    cache.append(torch.arange(T, device=DEV), k_bshd[:, :T], v_bshd[:, :T], attn.planes)
    q = cu(inp.q)
    out = torch.empty_like(q)
    step = ops.DecodeStep(cache, q, k_bshd[:, T:T + 1].contiguous(), v_bshd[:, T:T + 1].contiguous(),
                          torch.tensor([T], device=DEV), attn.planes, attn.protos_T, out, topk=M, sink=sink,
                          window=window, T_max=T + 64, keep_list=True)
    step.run()
    torch.cuda.synchronize()
    assert int(step.status) == 0 and int(cache.prefill_len) == T + 1
    # oracle on the same cache contents
    codes = cache.k_hard[:, :, :T + 1].cpu()
    vn = cache.v_norm[:, :, :T + 1].cpu()
    exact, _ = orc.hard_hash_keys_exact(inp.k.float().permute(0, 2, 1, 3), inp.planes.float())
    assert torch.equal(codes.to(torch.int16), exact.permute(0, 2, 1, 3))
    res = orc.decode_step(inp.q.float(), inp.k.float(), inp.v.float(), codes, vn, inp.planes.float(),
                          inp.protos_T, sink, window, M)
    ktot = res["sparse_list"].shape[-1]
    lst = step.list.cpu()[:, :, :ktot]
    assert (step.list_len.cpu() == ktot).all()
    # selection was made on this kernel's own scores; compare the sets where the oracle's
    # cut is clear of rounding-level near-ties, and the attention output always
    s = res["scores"].numpy()
    for b in range(B):
        for h in range(H):
            want = set(res["sparse_list"][b, h].tolist())
            got = set(lst[b, h].tolist())
            if want != got:
                diff = np.array(sorted(want ^ got))
                kth = np.sort(s[b, h])[::-1][M - 1]
                assert (np.abs(s[b, h][diff] - kth) <= 2e-5 * abs(kth)).all()
    assert (out.float().cpu() - res["out"].float()).abs().max() <= OUT_ATOL[dtype]
    # a second run of the same step object is idempotent on the cache and reproduces the output
    out1 = out.clone()
    step.run()
    torch.cuda.synchronize()
    assert torch.equal(out, out1)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_decode_step_packed_and_fp32_tables_agree(dtype):
    """The whole step with the list built from the packed 12-bit table against the step pinned to
    the fp32 table: same index sets, outputs within rounding of the summation order, over a few
    growing-context steps (the newest token must be scored in both)."""
    B, H, Hkv, T, M, sink, window = 2, 8, 2, 9000, 256, 8, 32
    inp = make_decode_inputs(B, H, Hkv, T + 4, seed=61, dtype=dtype)
    k_bshd = cu(inp.k.permute(0, 2, 1, 3).contiguous())
    v_bshd = cu(inp.v.permute(0, 2, 1, 3).contiguous())
    g = torch.Generator().manual_seed(3)
    qs = [cu(torch.randn(B, H, 128, generator=g).to(dtype)) for _ in range(4)]
    results = {}
    for path in ("filter_f32", "filter_packed"):
        attn = SocketAttention(H, Hkv, 128, heavy_const=M, sink_size=sink, window_size=window,
                               planes=inp.planes, protos_T=inp.protos_T, dtype=dtype, device=DEV)
        cache = attn.setup_cache(B, T + 64, dtype=dtype)
        cache.append(torch.arange(T, device=DEV), k_bshd[:, :T], v_bshd[:, :T], attn.planes)
        q = torch.empty(B, H, 128, dtype=dtype, device=DEV)
        kn = torch.empty(B, 1, Hkv, 128, dtype=dtype, device=DEV)
        vn = torch.empty_like(kn)
        pos = torch.zeros(1, dtype=torch.long, device=DEV)
        out = torch.empty_like(q)
        step = ops.DecodeStep(cache, q, kn, vn, pos, attn.planes, attn.protos_T, out, topk=M, sink=sink,
                              window=window, T_max=T + 64, keep_list=True, select_path=path)
        res = []
        for i in range(4):
            q.copy_(qs[i]); kn.copy_(k_bshd[:, T + i:T + i + 1]); vn.copy_(v_bshd[:, T + i:T + i + 1]); pos.fill_(T + i)
            step.run()
            torch.cuda.synchronize()
            res.append((torch.sort(step.list.clone(), dim=-1).values, step.list_len.clone(), out.clone()))
        assert int(step.status) == 0 and step.rescored_rows() == 0
        results[path] = res
    for (la, na, oa), (lb, nb_, ob) in zip(results["filter_f32"], results["filter_packed"]):
        assert torch.equal(na, nb_) and torch.equal(la, lb)
        assert (oa.float() - ob.float()).abs().max() <= (2e-3 if dtype == torch.bfloat16 else 1e-5)


def test_sparse_decode_rereads_non_contiguous_inputs_on_every_call():
    """The reference flow hands `v` over as a view of the fused QKV projection (not contiguous for
    B > 1).  Two calls with the same buffers and different contents must each use the contents of
    their own call; the result must equal the one obtained with contiguous copies."""
    B, H, Hkv, T, M, sink, window = 2, 8, 2, 2500, 64, 4, 16
    inp = make_decode_inputs(B, H, Hkv, T + 2, seed=31, dtype=torch.bfloat16)
    k_bshd = cu(inp.k.permute(0, 2, 1, 3).contiguous())
    v_bshd = cu(inp.v.permute(0, 2, 1, 3).contiguous())
    g = torch.Generator().manual_seed(8)
    qs = [cu(torch.randn(B, H, 128, generator=g).bfloat16()) for _ in range(2)]

    def run(contiguous):
        attn = SocketAttention(H, Hkv, 128, heavy_const=M, sink_size=sink, window_size=window,
                               planes=inp.planes, protos_T=inp.protos_T, dtype=torch.bfloat16, device=DEV)
        cache = attn.setup_cache(B, T + 64)
        cache.append(torch.arange(T, device=DEV), k_bshd[:, :T], v_bshd[:, :T], attn.planes)
        # one projection buffer [B, 1, (H + 2 Hkv) * D]; q, k, v are views of it, as in the reference
        qkv = torch.zeros(B, 1, (H + 2 * Hkv) * 128, dtype=torch.bfloat16, device=DEV)
        qv, kv, vv = qkv.split([H * 128, Hkv * 128, Hkv * 128], dim=-1)
        qv, kv, vv = qv.view(B, H, 128), kv.view(B, 1, Hkv, 128), vv.view(B, 1, Hkv, 128)
        assert not vv.is_contiguous() and not kv.is_contiguous()
        pos = torch.zeros(1, dtype=torch.long, device=DEV)
        outs = []
        for i in range(2):
            qv.copy_(qs[i]); kv.copy_(k_bshd[:, T + i:T + i + 1]); vv.copy_(v_bshd[:, T + i:T + i + 1])
            pos.fill_(T + i)
            if contiguous:
                o = attn.sparse_decode(qv.contiguous(), kv.contiguous(), vv.contiguous(), pos)
            else:
                o = attn.sparse_decode(qv, kv, vv, pos)
            outs.append(o.clone())
        torch.cuda.synchronize()
        assert int(cache.prefill_len) == T + 2 and int(cache.status) == 0
        return outs, cache.k_cache[:, :, T:T + 2].clone(), cache.v_cache[:, :, T:T + 2].clone()

    want, wk, wv = run(True)
    got, gk, gv = run(False)
    assert torch.equal(gk, wk) and torch.equal(gv, wv)
    assert torch.equal(gv, v_bshd[:, T:T + 2].permute(0, 2, 1, 3))
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    assert not torch.equal(got[0], got[1])


@pytest.mark.parametrize("ratio,T", [(0.03, 9000), (0.1, 5000), (0.0001, 4100)])
def test_budget_as_a_fraction_of_the_live_length(ratio, T):
    """`heavy_const` as a float is that fraction of the cached keys (the reference's
    `_effective_size`): each step must give what a module built with that step's integer budget
    gives, while the budget moves with the length from one call to the next (through both select
    paths: 3 % is inside the filtering scorer's range, 10 % is not)."""
    B, H, Hkv, sink, window = 1, 8, 2, 4, 16
    inp = make_decode_inputs(B, H, Hkv, T + 3, seed=77, dtype=torch.bfloat16)
    k_bshd = cu(inp.k.permute(0, 2, 1, 3).contiguous())
    v_bshd = cu(inp.v.permute(0, 2, 1, 3).contiguous())
    g = torch.Generator().manual_seed(9)
    qs = [cu(torch.randn(B, H, 128, generator=g).bfloat16()) for _ in range(3)]

    def run(budget_of_step):
        outs = []
        for i in range(3):
            attn = SocketAttention(H, Hkv, 128, heavy_const=budget_of_step(i), sink_size=sink, window_size=window,
                                   planes=inp.planes, protos_T=inp.protos_T, dtype=torch.bfloat16, device=DEV)
            cache = attn.setup_cache(B, T + 64)
            cache.append(torch.arange(T + i, device=DEV), k_bshd[:, :T + i], v_bshd[:, :T + i], attn.planes)
            pos = torch.tensor([T + i], dtype=torch.long, device=DEV)
            outs.append(attn.sparse_decode(qs[i], k_bshd[:, T + i:T + i + 1].contiguous(),
                                           v_bshd[:, T + i:T + i + 1].contiguous(), pos).clone())
            torch.cuda.synchronize()
            assert int(cache.status) == 0
        return outs

    want = run(lambda i: max(0, min(int(ratio * (T + i + 1)), T + i + 1)))
    # one module, one cache, the budget following the length; `pos` given on the host for the
    # first two calls and read back from the device for the third
    attn = SocketAttention(H, Hkv, 128, heavy_const=ratio, sink_size=sink, window_size=window,
                           planes=inp.planes, protos_T=inp.protos_T, dtype=torch.bfloat16, device=DEV)
    cache = attn.setup_cache(B, T + 64)
    cache.append(torch.arange(T, device=DEV), k_bshd[:, :T], v_bshd[:, :T], attn.planes)
    pos = torch.zeros(1, dtype=torch.long, device=DEV)
    budgets = []
    for i in range(3):
        pos.fill_(T + i)
        o = attn.sparse_decode(qs[i], k_bshd[:, T + i:T + i + 1].contiguous(), v_bshd[:, T + i:T + i + 1].contiguous(),
                               pos, pos=(T + i) if i < 2 else None)
        torch.cuda.synchronize()
        budgets.append(int(attn._step[1].params.M))
        assert torch.equal(o, want[i]), (ratio, T, i)
    assert budgets == [attn.effective_size(T + i + 1) for i in range(3)]
    assert int(cache.status) == 0 and int(cache.prefill_len) == T + 3


def test_run_to_run_determinism():
    inp = make_decode_inputs(1, 32, 8, 8192, seed=5, dtype=torch.bfloat16)
    qp = orc.soft_hash(inp.q.float(), inp.planes.float(), inp.protos_T)
    codes = ops.hash_keys(cu(inp.k), cu(inp.planes))
    vn = cu(orc.value_norm(inp.v.float()))
    outs = []
    for _ in range(3):
        lst, ln, sc = build_sparse_list_native(cu(qp), codes, vn, 8192, 16, 32, 512, return_scores=True)
        o = sparse_attention_fwd(cu(inp.q), cu(inp.k), cu(inp.v), lst, ln)
        outs.append((lst.clone(), sc.clone(), o.clone()))
    for a in outs[1:]:
        assert all(torch.equal(x, y) for x, y in zip(a, outs[0]))


# ---------------------------------------------------------------------------- fused scorer + select
def _fused_lists(q, planes, codes_d, vn_d, H, Hkv, T, M, sink, window, T_dev=None):
    """The fused scorer + select through every table form the shape allows: the fp32 table, and the
    packed 12-bit table where there is one.  Yields (name, lut, list, list_len, rescored rows)."""
    _, lut = ops.soft_hash(cu(q), cu(planes), cu(hypercube_protos(8)), 1.0, n_kv_heads=Hkv,
                           want_probs=False, want_lut=True)
    got, got_len, ws = ops.score_select_list(lut, codes_d, vn_d, H, T, M, sink, window, T_dev=T_dev)
    yield "fp32", lut, got, got_len, int(ws[:4].view(torch.int32).item())
    if ops.packed_applicable(q.shape[0], H, Hkv, 32, 256, T, M):
        lut2, packed = ops.soft_hash_packed(cu(q), cu(planes), cu(hypercube_protos(8)), 1.0, n_kv_heads=Hkv)
        assert torch.equal(lut2, lut)
        got, got_len, ws = ops.score_select_packed(lut2, packed, codes_d, vn_d, H, T, M, sink, window, T_dev=T_dev)
        yield "packed", lut, got, got_len, int(ws[:4].view(torch.int32).item())


def _fused_vs_two_step(B, H, Hkv, T, M, sink, window, v_norm=None, seed=0, Tcap=None):
    g = torch.Generator().manual_seed(seed)
    Tcap = Tcap or T
    q = torch.randn(B, H, 128, generator=g)
    planes = torch.randn(32, 8, 128, generator=g)
    codes = torch.randint(0, 256, (B, Hkv, Tcap, 32), generator=g, dtype=torch.uint8)
    if v_norm is None:
        v_norm = (torch.rand(B, Hkv, Tcap, generator=g) + 10.5).to(torch.float16)
    codes_d, vn_d = cu(codes), cu(v_norm.contiguous())
    n_resc = 0
    for name, lut, got, got_len, resc in _fused_lists(q, planes, codes_d, vn_d, H, Hkv, T, M, sink, window):
        scores = ops.score(lut, codes_d, vn_d, H, T)
        want, want_len = ops.select_list(scores, T, M, sink, window)
        assert torch.equal(got_len, want_len), name
        nb = got.shape[-1] - min(M, T)
        assert torch.equal(got[:, :, :nb], want[:, :, :nb]), name
        assert torch.equal(torch.sort(got[:, :, nb:], dim=-1).values, torch.sort(want[:, :, nb:], dim=-1).values), name
        # and the selection is a true top-k of the scores
        vals = torch.sort(torch.gather(scores, 2, got[:, :, nb:].long()), dim=-1, descending=True).values
        assert torch.equal(vals, torch.topk(scores[:, :, :T], min(M, T), dim=-1).values), name
        n_resc = max(n_resc, resc)
    return n_resc


@pytest.mark.parametrize("B,H,Hkv,T,M", [(1, 32, 8, 32768, 1024), (2, 8, 2, 20000, 512), (1, 4, 1, 4096, 64),
                                         (1, 8, 8, 9000, 100), (4, 32, 8, 131072, 2048), (1, 16, 2, 50001, 1)])
def test_fused_score_select_equals_two_step(B, H, Hkv, T, M):
    assert ops.score_select_applicable(B, H, Hkv, 32, 256, T, M)
    n_fallback = _fused_vs_two_step(B, H, Hkv, T, M, 8, 24, seed=T + M)
    assert n_fallback == 0          # benign rows are decided on the candidates alone


def test_fused_score_select_falls_back_exactly_on_hostile_rows():
    T = 40000
    ramp = (1.0 + 6.0 * torch.arange(T) / T).to(torch.float16)          # scores grow with position
    n1 = _fused_vs_two_step(1, 8, 2, T, 512, 4, 4, v_norm=ramp.expand(1, 2, T), seed=1)
    block = torch.ones(T)
    block[12000:15000] = 50.0                                           # one chunk holds all winners
    n2 = _fused_vs_two_step(1, 8, 2, T, 1024, 4, 4, v_norm=block.to(torch.float16).expand(1, 2, T), seed=2)
    flat = torch.ones(1, 2, T, dtype=torch.float16)
    codes_equal = _fused_vs_two_step(1, 8, 2, T, 256, 0, 0, v_norm=flat, seed=3)
    # a ramp and a block of winners no longer defeat the cut (it comes from a sample of the whole
    # row); whichever rows still take the rescoring path, the lists above were exact
    assert n1 >= 0 and n2 >= 0 and codes_equal >= 0


@pytest.mark.parametrize("B,H,Hkv,T,M", [(1, 32, 8, 131072, 2048), (4, 32, 8, 131072, 2048), (1, 32, 8, 32768, 1024)])
def test_fused_score_select_recent_keys_scoring_high_stay_on_the_candidate_path(B, H, Hkv, T, M):
    # the few hundred keys just before the query score far above the rest, as they do in a real model
    # (rotary embedding, local context), on top of a mild growth over the whole row.  The newest keys
    # are kept unfiltered and the cut comes from a sample of the whole row, so no run overflows and no
    # chunk cuts above the k-th score
    w = torch.linspace(0.0, 1.0, T)
    vn = 8.0 * (1.0 + 0.04 * w)                              # about one standard deviation of the scores
    vn[-700:] *= 3.0
    vn[:40] *= 3.0                                           # and a few "sink" keys at the start
    vn = vn.to(torch.float16).expand(B, Hkv, T)
    assert _fused_vs_two_step(B, H, Hkv, T, M, 64, 256, v_norm=vn, seed=T + B) == 0


@pytest.mark.parametrize("T", [131072 + 55, 131072 + 105, 131072 - 1, 130000])
def test_fused_score_select_short_segments_stay_on_the_candidate_path(T):
    # context lengths at which scorer CTAs straddle a KV-head boundary with a few hundred keys on
    # one side: the cut of such a short segment comes from one or two warps' samples and must still
    # stay below the row's k-th score
    assert _fused_vs_two_step(4, 32, 8, T, 2048, 64, 256, seed=T) == 0


@pytest.mark.parametrize("extra", [40, 300, 700, 1500, 5000])
def test_fused_score_select_live_length_just_past_a_cta_boundary(extra):
    # 128K-sized problem, flat split: the live length (device value) ends `extra` keys after the start
    # of some CTA's segment, so that CTA has a short live segment inside a long slot range
    B, H, Hkv, M, Tcap = 4, 32, 8, 2048, 131072 + 600
    per_cta = ((32 * (Tcap + 3584) + 147) // 148 + 31) // 32 * 32
    T_live = 4 * per_cta + extra
    g = torch.Generator().manual_seed(extra)
    q = torch.randn(B, H, 128, generator=g)
    planes = torch.randn(32, 8, 128, generator=g)
    codes = cu(torch.randint(0, 256, (B, Hkv, Tcap, 32), generator=g, dtype=torch.uint8))
    vn = cu((torch.rand(B, Hkv, Tcap, generator=g) + 10.5).to(torch.float16))
    T_dev = torch.tensor(T_live, dtype=torch.int32, device=DEV)
    for name, lut, got, got_len, resc in _fused_lists(q, planes, codes, vn, H, Hkv, Tcap, M, 64, 256, T_dev=T_dev):
        assert resc == 0, name                                 # no row went through the rescoring path
        scores = ops.score(lut, codes, vn, H, T_live)
        want, want_len = ops.select_list(scores, T_live, M, 64, 256)
        k = want.shape[-1]
        assert (got_len == k).all(), name
        assert torch.equal(torch.sort(got[:, :, :k], dim=-1).values, torch.sort(want, dim=-1).values), name


@pytest.mark.parametrize("B,H,Hkv,Tcap,T_live,M", [(1, 32, 8, 65536, 32768, 1024), (1, 2, 1, 50001, 25592, 512),
                                                   (2, 8, 2, 40000, 14000, 256)])
def test_fused_score_select_capacity_well_above_the_live_length(B, H, Hkv, Tcap, T_live, M):
    # the plan (chunks, run capacity) is made for the capacity; the kept fraction must follow the live
    # length, or the cut lands above the k-th score and every row is rescored
    g = torch.Generator().manual_seed(Tcap + M)
    q = torch.randn(B, H, 128, generator=g)
    planes = torch.randn(32, 8, 128, generator=g)
    codes = cu(torch.randint(0, 256, (B, Hkv, Tcap, 32), generator=g, dtype=torch.uint8))
    vn = cu((torch.rand(B, Hkv, Tcap, generator=g) + 10.5).to(torch.float16))
    T_dev = torch.tensor(T_live, dtype=torch.int32, device=DEV)
    for name, lut, got, got_len, resc in _fused_lists(q, planes, codes, vn, H, Hkv, Tcap, M, 8, 24, T_dev=T_dev):
        assert resc == 0, name
        scores = ops.score(lut, codes, vn, H, T_live)
        want, want_len = ops.select_list(scores, T_live, M, 8, 24)
        k = want.shape[-1]
        assert (got_len == k).all(), name
        assert torch.equal(torch.sort(got[:, :, :k], dim=-1).values, torch.sort(want, dim=-1).values), name


def test_fused_score_select_long_runs():
    # >= 128 keys per scorer warp, benign and hostile score layouts
    T = 140000
    n0 = _fused_vs_two_step(1, 8, 2, T, 1024, 8, 24, seed=11)
    assert n0 == 0
    ramp = (1.0 + 6.0 * torch.arange(T) / T).to(torch.float16)
    n1 = _fused_vs_two_step(1, 8, 2, T, 512, 4, 4, v_norm=ramp.expand(1, 2, T), seed=12)
    block = torch.ones(T)
    block[60000:66000] = 50.0
    n2 = _fused_vs_two_step(1, 8, 2, T, 1024, 4, 4, v_norm=block.to(torch.float16).expand(1, 2, T), seed=13)
    assert n1 >= 0 and n2 > 0        # 6000 winners in a row overflow their runs: the rescoring path ran, exactly
    # tiny and huge weights side by side: bounds in the half-precision subnormal range and near its top
    g = torch.Generator().manual_seed(14)
    mixed = torch.where(torch.rand(1, 2, T, generator=g) < 0.5, torch.full((1, 2, T), 3e-5),
                        torch.full((1, 2, T), 900.0)).to(torch.float16)
    _fused_vs_two_step(1, 8, 2, T, 700, 2, 2, v_norm=mixed, seed=15)
    _fused_vs_two_step(2, 32, 8, 300000, 2048, 64, 256, seed=16)


def test_fused_score_select_device_length_and_capacity():
    T_live, Tcap = 30000, 33000
    g = torch.Generator().manual_seed(9)
    B, H, Hkv, M = 1, 8, 2, 300
    q = torch.randn(B, H, 128, generator=g)
    planes = torch.randn(32, 8, 128, generator=g)
    codes = cu(torch.randint(0, 256, (B, Hkv, Tcap, 32), generator=g, dtype=torch.uint8))
    vn = cu((torch.rand(B, Hkv, Tcap, generator=g) + 1).to(torch.float16))
    T_dev = torch.tensor(T_live, dtype=torch.int32, device=DEV)
    for name, lut, got, got_len, _ in _fused_lists(q, planes, codes, vn, H, Hkv, Tcap, M, 4, 16, T_dev=T_dev):
        scores = ops.score(lut, codes, vn, H, T_live)
        want, want_len = ops.select_list(scores, T_live, M, 4, 16)
        k = want.shape[-1]
        assert (got_len == k).all(), name
        assert torch.equal(torch.sort(got[:, :, :k], dim=-1).values, torch.sort(want, dim=-1).values), name


@pytest.mark.parametrize("proto_kind,temperature,q_scale", [("corners", 0.3, 1.0), ("corners", 3.0, 0.05),
                                                             ("gauss", 1.0, 1.0), ("tiny", 1.0, 1.0),
                                                             ("gauss", 0.3, 0.2), ("wide", 1.0, 1.0)])
def test_packed_score_select_other_tables(proto_kind, temperature, q_scale):
    """The packed table's range comes from protos_T and the temperature alone: sharply peaked
    tables (low temperature, wide prototypes), nearly flat ones (the reference's 0.02-scaled
    initialisation) and unsaturated tanh (small queries) must all give the two-step list."""
    B, H, Hkv, T, M, sink, window = 2, 8, 2, 24000, 384, 8, 24
    g = torch.Generator().manual_seed(7 * len(proto_kind) + int(10 * temperature))
    q = torch.randn(B, H, 128, generator=g) * q_scale
    planes = torch.randn(32, 8, 128, generator=g)
    protos = {"corners": hypercube_protos(8), "gauss": torch.randn(8, 256, generator=g) * 0.5,
              "tiny": torch.randn(8, 256, generator=g) * 0.02,
              "wide": torch.randn(8, 256, generator=g) * 6.0}[proto_kind]
    codes = cu(torch.randint(0, 256, (B, Hkv, T, 32), generator=g, dtype=torch.uint8))
    vn = cu((torch.rand(B, Hkv, T, generator=g) + 10.5).to(torch.float16))
    lut, packed = ops.soft_hash_packed(cu(q), cu(planes), cu(protos), temperature, n_kv_heads=Hkv)
    _, lut_ref = ops.soft_hash(cu(q), cu(planes), cu(protos), temperature, n_kv_heads=Hkv, want_probs=False,
                               want_lut=True)
    assert torch.equal(lut, lut_ref)
    got, got_len, ws = ops.score_select_packed(lut, packed, codes, vn, H, T, M, sink, window)
    scores = ops.score(lut, codes, vn, H, T)
    want, want_len = ops.select_list(scores, T, M, sink, window)
    nb = want.shape[-1] - M
    assert torch.equal(got_len, want_len)
    assert torch.equal(got[:, :, :nb], want[:, :, :nb])
    assert torch.equal(torch.sort(got[:, :, nb:], dim=-1).values, torch.sort(want[:, :, nb:], dim=-1).values)


def test_packed_table_entries_bound_the_fp32_table():
    """Every 12-bit entry e of the packed table satisfies e <= (p - lo) * C < e + 1 for one (lo, C)
    per call: recovered here from the entries themselves, the relation must hold with a slack far
    below one unit, and no entry may sit at the clamps."""
    B, H, Hkv = 1, 8, 2
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, H, 128, generator=g)
    planes = torch.randn(32, 8, 128, generator=g)
    lut, packed = ops.soft_hash_packed(cu(q), cu(planes), cu(hypercube_protos(8)), 1.0, n_kv_heads=Hkv)
    groups = B * Hkv
    ent = packed[:groups * 65536].view(torch.int16).view(groups, 256, 32, 4).cpu().long()     # [g][r][l][head]
    p = lut.view(groups, 256, 32, 4).cpu().double()
    assert ent.min() > 0 and ent.max() < 4095
    # least squares for entry + 0.5 ~ (p - lo) * C, then the residual must stay inside half a unit
    x, y = p.flatten(), ent.flatten().double() + 0.5
    C = ((x - x.mean()) * (y - y.mean())).sum() / ((x - x.mean()) ** 2).sum()
    lo = x.mean() - y.mean() / C
    resid = (p - lo) * C - ent.double()
    assert resid.min() > -0.05 and resid.max() < 1.05
    K0 = packed[groups * 65536:groups * 65536 + 4 * groups].view(torch.float32).cpu().double()
    assert torch.allclose(K0, 32 * lo * C * torch.ones_like(K0), rtol=1e-3)


# ---------------------------------------------------------------------------- one-launch scorer + select (clusters)
def _cluster_vs_two_step(B, H, Hkv, T, M, sink, window, v_norm=None, codes=None, seed=0, Tcap=None, T_live=None):
    g = torch.Generator().manual_seed(seed)
    Tcap = Tcap or T
    q = torch.randn(B, H, 128, generator=g)
    planes = torch.randn(32, 8, 128, generator=g)
    if codes is None:
        codes = torch.randint(0, 256, (B, Hkv, Tcap, 32), generator=g, dtype=torch.uint8)
    if v_norm is None:
        v_norm = (torch.rand(B, Hkv, Tcap, generator=g) + 10.5).to(torch.float16)
    _, lut = ops.soft_hash(cu(q), cu(planes), cu(hypercube_protos(8)), 1.0, n_kv_heads=Hkv,
                           want_probs=False, want_lut=True)
    codes_d, vn_d = cu(codes.contiguous()), cu(v_norm.contiguous())
    T_eff = T if T_live is None else T_live
    T_dev = None if T_live is None else torch.tensor(T_live, dtype=torch.int32, device=DEV)
    scores = ops.score(lut, codes_d, vn_d, H, T_eff)
    want, want_len = ops.select_list(scores, T_eff, M, sink, window)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got, got_len = ops.score_select_cluster(lut, codes_d, vn_d, H, T, M, sink, window, T_dev=T_dev, status=status)
    assert int(status) == 0
    assert torch.equal(got_len, want_len)
    k = want.shape[-1]
    Me = min(M, T_eff)
    nb = k - Me
    assert torch.equal(got[:, :, :nb], want[:, :, :nb])
    heavy = got[:, :, nb:k]
    # exactly the two-step selection (ties included), and in ascending index order
    assert torch.equal(heavy, torch.sort(want[:, :, nb:], dim=-1).values)


@pytest.mark.parametrize("B,H,Hkv,T,M", [(1, 32, 8, 32768, 1024), (1, 32, 8, 33801, 1024), (2, 8, 2, 20000, 512),
                                         (1, 4, 1, 4096, 64), (1, 8, 2, 1000, 100), (1, 8, 2, 77, 200),
                                         (1, 16, 2, 50001, 1), (1, 8, 1, 81920, 4096), (1, 8, 2, 40, 40), (2, 32, 8, 20000, 512)])
def test_cluster_score_select_equals_two_step(B, H, Hkv, T, M):
    assert 2 <= ops.score_select_cluster_size(B, H, Hkv, 32, 256, T, M) <= 16
    _cluster_vs_two_step(B, H, Hkv, T, M, 8, 24, seed=T + M)


def test_cluster_score_select_ties_and_hostile_rows():
    T = 40000
    ramp = (1.0 + 6.0 * torch.arange(T) / T).to(torch.float16)          # scores grow with position
    _cluster_vs_two_step(1, 8, 2, T, 512, 4, 4, v_norm=ramp.expand(1, 2, T), seed=1)
    block = torch.ones(T)
    block[12000:15000] = 50.0                                           # one CTA holds all winners
    _cluster_vs_two_step(1, 8, 2, T, 1024, 4, 4, v_norm=block.to(torch.float16).expand(1, 2, T), seed=2)
    # all keys share their codes: every score of a row is equal, the lowest indices must win
    flat = torch.ones(1, 2, T, dtype=torch.float16)
    same = torch.randint(0, 256, (1, 2, 1, 32), dtype=torch.uint8).expand(1, 2, T, 32)
    _cluster_vs_two_step(1, 8, 2, T, 256, 0, 0, v_norm=flat, codes=same, seed=3)
    # a few distinct score levels with thousands of keys each: the boundary bin overflows the pairwise
    # ranking and is refined level by level down to exact ties
    few = torch.randint(0, 256, (1, 2, 4, 32), dtype=torch.uint8)
    pick = torch.randint(0, 4, (T,))
    _cluster_vs_two_step(1, 8, 2, T, 3000, 2, 2, v_norm=flat, codes=few[:, :, pick], seed=4)
    # zero value norms (score 0) mixed with live keys, fewer live keys than the budget
    vz = torch.zeros(1, 2, T, dtype=torch.float16)
    vz[:, :, ::97] = 2.0
    _cluster_vs_two_step(1, 8, 2, T, 1024, 4, 4, v_norm=vz, seed=5)


def test_cluster_score_select_device_length():
    _cluster_vs_two_step(1, 8, 2, 33000, 300, 4, 16, seed=9, T_live=30000)
    _cluster_vs_two_step(1, 8, 2, 33000, 300, 4, 16, seed=10, T_live=1)
    _cluster_vs_two_step(1, 8, 2, 33000, 300, 4, 16, seed=11, T_live=257)


def test_cluster_score_select_rejects_shapes_outside_its_range():
    assert ops.score_select_cluster_size(4, 32, 8, 32, 256, 131072, 2048) == 0      # keys per CTA
    assert ops.score_select_cluster_size(1, 8, 8, 32, 256, 8192, 100) == 0          # one head per KV head
    assert ops.score_select_cluster_size(1, 32, 8, 16, 256, 8192, 100) == 0         # L
    lut = torch.zeros(8 * 32 * 256, device=DEV)
    codes = torch.zeros(1, 8, 8192, 32, dtype=torch.uint8, device=DEV)
    vn = torch.ones(1, 8, 8192, dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError, match="outside the one-launch path"):
        ops.score_select_cluster(lut, codes, vn, 8, 8192, 100, 4, 4)


# ---------------------------------------------------------------------------- tensor-core bulk hashing
def test_tensor_core_hashing_is_bit_exact():
    g = torch.Generator().manual_seed(31)
    N = 5000 + 37
    planes = torch.randn(32, 8, 128, generator=g).bfloat16()
    keys = (torch.randn(N, 128, generator=g) * torch.exp(torch.randn(128, generator=g))).bfloat16()
    keys[5] = 0                                            # a zero row: every projection is exactly 0
    keys[6] = 0
    keys[6, 0], keys[6, 1] = planes[3, 2, 1], -planes[3, 2, 0]   # exactly orthogonal to plane (3,2)
    keys[7] = planes[10, 4] * 1e-3                         # tiny but parallel to a plane
    keys[8] = -planes[10, 4]
    keys[100:200] *= 1e-20                                 # very small magnitudes
    keys[200:300] *= 1e18
    want, _ = orc.hard_hash_keys_exact(keys.float()[None, :, None, :], planes.float())
    want = want[0, :, 0].to(torch.uint8)
    got = ops.hash_keys_tc(cu(keys), cu(planes)).cpu()
    assert torch.equal(got, want)
    assert torch.equal(ops.hash_keys(cu(keys), cu(planes)).cpu(), want)
    assert (got[5] == 255).all()


def test_tensor_core_hashing_pipeline_over_many_tiles():
    """Enough rows that every persistent CTA walks several tiles, so that the load / multiply /
    epilogue pipeline and its barriers go round many times: no wait may run out (status stays 0, and
    the call takes milliseconds, not the seconds a timed-out wait costs), and the codes equal the
    exact kernel's."""
    g = torch.Generator().manual_seed(35)
    N = 148 * 128 * 9 + 77
    planes = cu(torch.randn(32, 8, 128, generator=g).bfloat16())
    keys = cu((torch.randn(N, 128, generator=g) * torch.exp(0.5 * torch.randn(128, generator=g))).bfloat16())
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.hash_keys_tc(keys, planes, status=status)                  # warm-up (tensor maps, attributes)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    got = ops.hash_keys_tc(keys, planes, status=status)
    e1.record()
    torch.cuda.synchronize()
    assert int(status) == 0
    assert e0.elapsed_time(e1) < 50.0, e0.elapsed_time(e1)
    assert torch.equal(got, ops.hash_keys(keys, planes))


def test_tensor_core_hashing_overflow_path_is_exact():
    # every key exactly orthogonal to many planes: the near-zero list overflows and the exact
    # rehash takes over
    g = torch.Generator().manual_seed(32)
    planes = torch.randn(32, 8, 128, generator=g).bfloat16()
    planes[:, :, 64:] = 0
    N = 6000
    keys = torch.zeros(N, 128)
    keys[:, 64:] = torch.randn(N, 64, generator=g)         # support disjoint from the planes: all dots are 0
    keys = keys.bfloat16()
    got = ops.hash_keys_tc(cu(keys), cu(planes)).cpu()
    assert (got == 255).all()
