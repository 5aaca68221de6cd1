"""Generate the golden fixtures by running the REFERENCE's own code on CPU.

Run once, in a container that has the reference tree (a `reference` directory beside this repository, override
with SOCKET_REFERENCE_ROOT):

    python tests/golden/make_golden.py

What is executed from the reference (nothing of it is copied into this repository):
  * `Attention.hard_hash_keys`, `Attention.soft_hash`, `KVCache.update`,
    `Attention.sparse_forward`           (GPT-FAST/model.py)
  * the scorer kernel source compiled as host C++ (oracle/build_oracle.py -> oracle/_ref)
  * `build_sparse_list_decode` and `sparse_attention_fwd` (GPT-FAST/kernels/sparse.py): their
    source text is loaded at run time with the `.is_cuda` assertions dropped, the CUDA
    extension handle replaced by the host-compiled scorer, and the Triton kernels executed
    by the Triton interpreter (TRITON_INTERPRET=1).
The results are frozen as .npz files next to this script; `tests/test_oracle_golden.py`
checks the CPU oracle against them and the GPU tests check the CUDA kernels against them.
"""
from __future__ import annotations

import hashlib
import inspect
import math
import os
import re
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("SOCKET_REFERENCE_ROOT") or os.path.normpath(os.path.join(ROOT, "..", "reference"))
sys.path.insert(0, os.path.join(REF, "GPT-FAST"))
sys.path.insert(0, ROOT)

import model as refmodel                      # noqa: E402  (reference)
from kernels import sparse as refsparse       # noqa: E402  (reference)

from oracle import c_oracle                   # noqa: E402
from socket_b200.synth import hypercube_protos, make_decode_inputs  # noqa: E402


class _HostScorerExt:
    """Stands where the reference's JIT-compiled CUDA extension stands; runs the same kernel
    source on the host."""

    @staticmethod
    def soft_hash_collision(q_probs, key_buckets, allowed_ext, v_hist):
        return c_oracle.ref_soft_hash_collision(q_probs, key_buckets, allowed_ext, v_hist)


def _cpu_capable(fn):
    """Re-create a reference function from its own source with the device assertions
    removed, inside the reference module's namespace."""
    src = inspect.getsource(fn)
    src = "\n".join(line for line in src.splitlines() if ".is_cuda" not in line)
    src = re.sub(r"^@torch\.no_grad\(\)\n", "", src, flags=re.M)
    ns = dict(refsparse.__dict__)
    ns["_get_soft_hash_ext"] = lambda: _HostScorerExt
    exec(compile(src, f"<reference {fn.__name__}>", "exec"), ns)
    return ns[fn.__name__]


ref_build_list = _cpu_capable(refsparse.build_sparse_list_decode)
ref_sparse_fwd = _cpu_capable(refsparse.sparse_attention_fwd)


def make_attention(H, Hkv, D, L, P, M, planes, protos_T):
    cfg = refmodel.ModelArgs(n_layer=1, n_head=H, dim=H * D, n_local_heads=Hkv, L=L, K=P,
                             R=1 << P, heavy_const=M, vocab_size=64)
    attn = refmodel.Attention(cfg)
    with torch.no_grad():
        attn.planes.copy_(planes.float())
        attn.protos_T.copy_(protos_T.float())
    return attn, cfg


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def run_ops(inp, sink, window, M, allowed=None, temperature=1.0):
    """Operator-level reference run on canonical inputs (fp32 tensors holding the
    possibly bf16-rounded values)."""
    q = inp.q.float()
    k = inp.k.float()
    v = inp.v.float()
    planes = inp.planes.float()
    B, H, D = q.shape
    _, Hkv, T, _ = k.shape
    L, P, _ = planes.shape
    rep = H // Hkv
    attn, _ = make_attention(H, Hkv, D, L, P, M, planes, inp.protos_T)
    with torch.no_grad():
        codes_bshl = attn.hard_hash_keys(k.permute(0, 2, 1, 3).contiguous())      # [B,T,Hkv,L]
        q_probs = attn.soft_hash(q)                                                # [B,H,L,R]
        if temperature != 1.0:
            raise NotImplementedError
        v_norm_bsh = torch.linalg.vector_norm(v.permute(0, 2, 1, 3).float(), ord=2, dim=-1).to(torch.float16)
        cache = refmodel.KVCache(B, T, Hkv, D, L=L, R=1 << P, dtype=torch.float32)
        cache.update(torch.arange(T), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3),
                     v_norm=v_norm_bsh, k_hard=codes_bshl)
        k_hard = cache.k_hard                                                      # [B,Hkv,T,L]
        k_hard_bhlt = k_hard.repeat_interleave(rep, dim=1).permute(0, 1, 3, 2).contiguous()
        v_norm_bht = cache.v_norm.repeat_interleave(rep, dim=1)
        if allowed is None:
            allowed = torch.ones(B, H, T, dtype=torch.bool)
        scores = c_oracle.ref_soft_hash_collision(
            q_probs.float().unsqueeze(2), k_hard_bhlt, allowed.unsqueeze(2),
            v_norm_bht.float().unsqueeze(2)).squeeze(2)
        sparse_list, sparse_len = ref_build_list(q_probs, k_hard_bhlt, v_norm_bht, allowed,
                                                 sink=sink, window=window, M=M)
        lst = sparse_list
        if (lst < 0).any():
            # the reference kernels would read row -1; golden attention output is taken on
            # the list with masked entries removed per row (equal-length rows not required)
            out = None
        else:
            out = ref_sparse_fwd(q, cache.k_cache, cache.v_cache, sparse_list, sparse_len)
    return dict(codes=k_hard.to(torch.int16), v_norm=cache.v_norm, q_probs=q_probs.float(),
                scores=scores, sparse_list=sparse_list, sparse_len=sparse_len, out=out,
                allowed=allowed)


def save_case(name, inp, res, sink, window, M, store_inputs=True, extra=None):
    d = dict(sink=np.int64(sink), window=np.int64(window), M=np.int64(M),
             meta=np.array(repr(inp.meta)))
    low = inp.q.dtype != torch.float32
    if store_inputs:
        for key in ("planes", "q", "k", "v"):
            t = getattr(inp, key)
            d["in_" + key] = (t.view(torch.int16).numpy() if low else t.numpy())
        d["in_protos_T"] = inp.protos_T.numpy()
        d["in_dtype"] = np.array(str(inp.q.dtype))
    else:
        d["in_sha_k"] = np.array(sha(inp.k.float()))
        d["in_sha_q"] = np.array(sha(inp.q.float()))
    d["codes_sha"] = np.array(res["codes_sha"])
    for key in ("codes", "v_norm", "q_probs", "scores", "sparse_list", "sparse_len", "out", "allowed"):
        t = res.get(key)
        if t is None:
            continue
        if key == "v_norm":
            d[key] = t.view(torch.int16).numpy()
        elif key == "codes":
            d[key] = t.to(torch.uint8).numpy()
        else:
            d[key] = t.numpy()
    if extra:
        d.update(extra)
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **d)
    print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB")


def case_ops(name, B, H, Hkv, T, sink, window, M, seed, dtype=torch.float32, mask_fn=None,
             store_inputs=True, drop=()):
    inp = make_decode_inputs(B, H, Hkv, T, seed=seed, dtype=dtype)
    allowed = mask_fn(B, H, T) if mask_fn else None
    res = run_ops(inp, sink, window, M, allowed=allowed)
    res["codes_sha"] = sha(res["codes"].to(torch.uint8))
    for key in drop:
        res[key] = None
    save_case(name, inp, res, sink, window, M, store_inputs=store_inputs)


def case_model_flow(name="model_flow"):
    """Whole `Attention.sparse_forward` of the reference: a dense prefill of S tokens that
    hashes and caches them, then one sparse decode step.  Captures the tensors at the
    operator boundary."""
    torch.manual_seed(7)
    B, H, Hkv, D, L, P, M = 1, 8, 2, 128, 32, 8, 24
    S, Tcap = 95, 128
    g = torch.Generator().manual_seed(77)
    planes = torch.randn(L, P, D, generator=g)
    protos = hypercube_protos(P)
    attn, cfg = make_attention(H, Hkv, D, L, P, M, planes, protos)
    cfg.sink_size, cfg.window_size = 4, 8
    attn.kv_cache = refmodel.KVCache(B, Tcap, Hkv, D, L=L, R=1 << P, dtype=torch.float32)
    freqs_all = refmodel.precompute_freqs_cis(Tcap, D, 500000)
    causal = torch.tril(torch.ones(Tcap, Tcap, dtype=torch.bool))
    cap = {}
    orig_soft, orig_hard = attn.soft_hash, attn.hard_hash_keys

    def soft(qb):
        cap["q"] = qb.clone()
        r = orig_soft(qb)
        cap["q_probs"] = r.clone()
        return r

    def hard(kb):
        cap.setdefault("k_calls", []).append(kb.clone())
        return orig_hard(kb)

    def build(*a, **kw):
        r = ref_build_list(*a, **kw)
        cap["sparse_list"], cap["sparse_len"] = r[0].clone(), r[1].clone()
        return r

    def fwd(*a, **kw):
        r = ref_sparse_fwd(*a, **kw)
        cap["out_bhd"] = r.clone()
        return r

    attn.soft_hash, attn.hard_hash_keys = soft, hard
    refmodel.build_sparse_list_decode, refmodel.sparse_attention_fwd = build, fwd
    with torch.no_grad():
        x = torch.randn(B, S, H * D, generator=g) * 0.5
        pos = torch.arange(S)
        attn.sparse_forward(x, freqs_all[pos], causal[None, None, pos], None, pos)
        x1 = torch.randn(B, 1, H * D, generator=g) * 0.5
        pos1 = torch.tensor([S])
        y = attn.sparse_forward(x1, freqs_all[pos1], causal[None, None, pos1], None, pos1)
    T = int(attn.kv_cache.prefill_len.item())
    d = dict(
        planes=planes.numpy(), protos_T=protos.numpy(), q=cap["q"].numpy(),
        k_prefill=cap["k_calls"][0].numpy(), k_step=cap["k_calls"][1].numpy(),
        k_cache=attn.kv_cache.k_cache.numpy(), v_cache=attn.kv_cache.v_cache.numpy(),
        codes=attn.kv_cache.k_hard.to(torch.uint8).numpy(),
        v_norm=attn.kv_cache.v_norm.view(torch.int16).numpy(),
        q_probs=cap["q_probs"].numpy(), sparse_list=cap["sparse_list"].numpy(),
        sparse_len=cap["sparse_len"].numpy(), out_bhd=cap["out_bhd"].numpy(),
        T=np.int64(T), S=np.int64(S), sink=np.int64(4), window=np.int64(8), M=np.int64(M))
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **d)
    print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB  (T={T})")


def main():
    def mask_sparse(B, H, T):
        g = torch.Generator().manual_seed(5)
        m = torch.rand(B, H, T, generator=g) < 0.2          # only ~20 % allowed
        m[..., 0] = False
        return m

    case_ops("tiny_rep4_f32", 1, 8, 2, 200, sink=4, window=8, M=32, seed=11)
    case_ops("tiny_rep4_bf16", 1, 8, 2, 200, sink=4, window=8, M=32, seed=12, dtype=torch.bfloat16)
    case_ops("batch2_rep4_f32", 2, 8, 2, 257, sink=3, window=5, M=40, seed=13, drop=("q_probs",))
    case_ops("edge_short_ctx", 1, 4, 1, 17, sink=20, window=5, M=32, seed=14, drop=("q_probs",))
    case_ops("edge_no_base", 1, 4, 2, 64, sink=0, window=0, M=8, seed=15, drop=("q_probs",))
    case_ops("edge_masked", 1, 4, 1, 100, sink=2, window=4, M=40, seed=16, mask_fn=mask_sparse,
             drop=("q_probs",))
    case_ops("rep1_mha", 1, 2, 2, 128, sink=2, window=6, M=16, seed=17, drop=("q_probs",))
    case_ops("rep8_gqa", 1, 8, 1, 128, sink=2, window=6, M=16, seed=18, drop=("q_probs",))
    case_ops("c1_config", 1, 32, 8, 4096, sink=16, window=64, M=256, seed=1234,
             store_inputs=False, drop=("codes", "q_probs", "v_norm"))
    case_model_flow()


if __name__ == "__main__":
    main()
