"""Host-side mirror of the SOCKET pieces of `GPT-FAST/model.py`: the KV cache with bucket
codes and value norms, the hash methods of `Attention`, and the decode branch of
`Attention.sparse_forward` between the QKV projection and the output projection."""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Union

import torch
import torch.nn as nn
from torch import Tensor

from . import ops


class KVCache(nn.Module):
    """KV is stored as (B, H, T, D), like the reference cache (GPT-FAST/model.py:157-185), with
    the per-key bucket codes `k_hard [B,H,T,L]` and value norms `v_norm [B,H,T]`.  Codes are
    uint8 (one byte per table, P <= 8) instead of the reference's int16."""

    def __init__(self, max_batch_size: int, max_seq_length: int, n_heads: int, head_dim: int,
                 L: int, R: int, dtype=torch.bfloat16, device=None):
        super().__init__()
        if R > 256:
            raise RuntimeError("socket_b200.KVCache stores uint8 codes: R must be <= 256")
        B, H, T, D = max_batch_size, n_heads, max_seq_length, head_dim
        self.register_buffer("k_cache", torch.zeros((B, H, T, D), dtype=dtype, device=device))
        self.register_buffer("v_cache", torch.zeros((B, H, T, D), dtype=dtype, device=device))
        self.L = L
        self.R = R
        self.register_buffer("k_hard", torch.zeros((B, H, T, L), dtype=torch.uint8, device=device))
        self.register_buffer("v_norm", torch.zeros((B, H, T), dtype=torch.float16, device=device))
        self.register_buffer("attn_out", torch.zeros((B, H, D), dtype=dtype, device=device))
        self.register_buffer("prefill_len", torch.zeros((), dtype=torch.int32, device=device))
        self.register_buffer("status", torch.zeros((), dtype=torch.int32, device=device))

    def append(self, input_pos: Tensor, k_val: Tensor, v_val: Tensor, planes: Tensor) -> None:
        """Fused path: hash `k_val`, take ||v||, write all four arrays and advance
        `prefill_len`, in one launch and without a host sync.  A position outside the cache
        is not written and sets bit SK_DEV_POS_OUT_OF_RANGE of `status`."""
        if input_pos.dtype != torch.long:
            input_pos = input_pos.long()
        ops.kv_append(self.k_cache, self.v_cache, self.k_hard, self.v_norm, self.prefill_len,
                      input_pos, k_val, v_val, planes, status=self.status)

    def update(self, input_pos: Tensor, k_val: Tensor, v_val: Tensor,
               v_norm: Optional[Tensor] = None, k_hard: Optional[Tensor] = None):
        """Same contract as the reference `KVCache.update` (GPT-FAST/model.py:187-229),
        including the host-side bounds check that raises RuntimeError; takes precomputed
        `v_norm [B,S,H]` / `k_hard [B,S,H,L]`.  Use `append` on the hot path."""
        if input_pos.dtype != torch.long:
            input_pos = input_pos.long()
        assert input_pos.ndim == 1, f"input_pos must be [S], got {tuple(input_pos.shape)}"
        S = int(input_pos.numel())
        assert k_val.ndim == 4 and v_val.ndim == 4
        assert k_val.shape[1] == S and v_val.shape[1] == S, "k/v S dim must match input_pos length"
        Tcap = self.k_cache.size(2)
        max_pos = int(input_pos.max().item()) if S > 0 else -1
        min_pos = int(input_pos.min().item()) if S > 0 else 0
        if max_pos >= Tcap or min_pos < 0:
            raise RuntimeError(
                f"KVCache.update out-of-bounds: input_pos in [{min_pos},{max_pos}] but cache T={Tcap}. "
                f"Did you call setup_caches(max_seq_length >= max(input_pos)+1)?")
        self.k_cache[:, :, input_pos, :] = k_val.permute(0, 2, 1, 3).to(self.k_cache.dtype)
        self.v_cache[:, :, input_pos, :] = v_val.permute(0, 2, 1, 3).to(self.v_cache.dtype)
        if v_norm is not None:
            self.v_norm[:, :, input_pos] = v_norm.permute(0, 2, 1).to(torch.float16)
        if k_hard is not None:
            self.k_hard[:, :, input_pos, :] = k_hard.permute(0, 2, 1, 3).to(torch.uint8)
        self.prefill_len.fill_(max(int(self.prefill_len.item()), max_pos + 1))
        return self.k_cache, self.v_cache


class SocketAttention(nn.Module):
    """The SOCKET state and methods of the reference `Attention` module
    (GPT-FAST/model.py:377-413, 482-552) without the projections around them.

    planes [L,P,D] and protos_T [P,R] are buffers, as in the reference; `heavy_const` is
    the top-k budget - an int, or a float for that fraction of the cached keys (eager
    `sparse_decode` only; see `effective_size`) - and `sink_size`/`window_size` the structured
    part of the list (model.py:511-513)."""

    def __init__(self, n_head: int, n_local_heads: int, head_dim: int, L: int = 32, P: int = 8,
                 heavy_const: Union[int, float] = 1024, sink_size: int = 64, window_size: int = 128,
                 temperature: float = 1.0, planes: Optional[Tensor] = None,
                 protos_T: Optional[Tensor] = None, dtype=torch.bfloat16, device=None):
        super().__init__()
        assert n_head % n_local_heads == 0
        self.n_head, self.n_local_heads, self.head_dim = n_head, n_local_heads, head_dim
        self.L, self.K, self.R = L, P, 1 << P
        self.heavy_const, self.sink_size, self.window_size = heavy_const, sink_size, window_size
        self.temperature = temperature
        if planes is None:
            planes = torch.randn(L, P, head_dim) * 0.02
        if protos_T is None:
            protos_T = torch.randn(P, 1 << P) * 0.02
        self.register_buffer("planes", planes.to(device=device, dtype=dtype))
        self.register_buffer("protos_T", protos_T.to(device=device, dtype=torch.float32))
        self.kv_cache: Optional[KVCache] = None
        self._step = None
        self._stage = None

    def setup_cache(self, max_batch_size: int, max_seq_length: int, dtype=torch.bfloat16) -> KVCache:
        self.kv_cache = KVCache(max_batch_size, max_seq_length, self.n_local_heads, self.head_dim,
                                L=self.L, R=self.R, dtype=dtype, device=self.planes.device)
        self._step = None
        return self.kv_cache

    # -- the three hash methods, same names and shapes as the reference --------------------
    def soft_hash(self, queries_bhd: Tensor) -> Tensor:
        """[B,H,D] -> q_probs [B,H,L,R] (GPT-FAST/model.py:392-401), computed in fp32."""
        probs, _ = ops.soft_hash(queries_bhd, self.planes, self.protos_T, self.temperature,
                                 n_kv_heads=self.n_local_heads)
        return probs

    def pack_bits(self, bits: Tensor) -> Tensor:
        """[..., P] bool -> int16, first plane most significant (GPT-FAST/model.py:403-407)."""
        P = bits.shape[-1]
        weights = (1 << torch.arange(P - 1, -1, -1, device=bits.device, dtype=torch.int16))
        return (bits.to(torch.int16) * weights.view((1,) * (bits.ndim - 1) + (P,))).sum(dim=-1)

    @torch.no_grad()
    def hard_hash_keys(self, keys_bshd: Tensor) -> Tensor:
        """[B,S,Hkv,D] -> int16 codes [B,S,Hkv,L] (GPT-FAST/model.py:409-413)."""
        return ops.hash_keys(keys_bshd, self.planes.to(keys_bshd.dtype), code_dtype=torch.int16)

    # -- decode branch of sparse_forward ---------------------------------------------------
    @torch.no_grad()
    def effective_size(self, n_keys: int) -> int:
        """The top-k budget for `n_keys` cached keys: `heavy_const` itself when it is an int, that
        fraction of the keys when it is a float (pipeline/train_quest/modeling/modeling_llama.py:645-648,
        806-808), clamped to [0, n_keys]."""
        m = int(self.heavy_const * n_keys) if isinstance(self.heavy_const, float) else int(self.heavy_const)
        return max(0, min(m, n_keys))

    def sparse_decode(self, q_bhd: Tensor, k_new: Tensor, v_new: Tensor, input_pos: Tensor,
                      out: Optional[Tensor] = None, pos: Optional[int] = None) -> Tensor:
        """One decode step: q [B,H,D]; k_new, v_new [B,1,Hkv,D]; input_pos [1] (device).
        Appends the token, builds the sparse list from the cache-native codes and attends;
        returns out [B,H,D].  No relayout, no prefix copy, no host sync - unless `heavy_const` is a
        fraction: the budget then follows the live length, which the caller passes as `pos` (the
        new token's position as a host integer, as the reference's eager path has it) or which is
        read back from `input_pos`."""
        cache = self.kv_cache
        assert cache is not None, "Call setup_cache() first so kv_cache exists"
        if input_pos.dtype != torch.long:
            input_pos = input_pos.long()
        if out is None:
            out = torch.empty(q_bhd.shape, dtype=q_bhd.dtype, device=q_bhd.device)
        Tcap = cache.k_cache.shape[2]
        # The step holds raw addresses.  Contiguous inputs are read in place; a non-contiguous one
        # (the reference flow hands over `v` as a view of the fused QKV projection) is copied, on
        # every call, into a staging tensor that lives as long as the step does - never into a
        # temporary behind the address cache.
        ins = [q_bhd, k_new, v_new]
        if self._stage is None or any(s.shape != t.shape or s.dtype != t.dtype or s.device != t.device
                                      for s, t in zip(self._stage, ins)):
            self._stage = [torch.empty(t.shape, dtype=t.dtype, device=t.device) for t in ins]
            self._step = None
        src = []
        for t, s in zip(ins, self._stage):
            if t.is_contiguous():
                src.append(t)
            else:
                s.copy_(t)
                src.append(s)
        key = tuple(t.data_ptr() for t in src) + (input_pos.data_ptr(), out.data_ptr())
        ratio = isinstance(self.heavy_const, float)
        if self._step is None:
            step = ops.DecodeStep(cache, src[0], src[1], src[2], input_pos, self.planes, self.protos_T, out,
                                  topk=self.effective_size(Tcap), sink=self.sink_size, window=self.window_size,
                                  T_max=Tcap, temperature=self.temperature)
            self._step = (key, step)
        elif self._step[0] != key:
            # other tensors of the same shapes: new addresses, same scratch memory
            self._step[1].rebind(src[0], src[1], src[2], input_pos, out)
            self._step = (key, self._step[1])
        if ratio:
            n_keys = (int(pos) if pos is not None else int(input_pos.item())) + 1
            self._step[1].set_topk(self.effective_size(n_keys))
        self._step[1].run()
        return out

    def host_decoder(self, batch: int) -> "HostDecodeStep":
        """A decode step fed from, and answering into, pinned host memory (see HostDecodeStep)."""
        return HostDecodeStep(self, batch)


class HostDecodeStep:
    """One decode step whose inputs live in host memory: a single pinned staging block
    `[input_pos | q | k_new | v_new]` goes to the device in one copy, the four kernels of
    `sk_decode_step` run, and the last of them writes the output straight into pinned host
    memory (it is mapped into the device's address space, so no copy node is needed) — all of it
    one CUDA graph, so a step costs one launch call.  Write the inputs through `h_q`, `h_k`,
    `h_v`, `h_pos` (views of the staging block) or hand a packed block to `stage()`, call
    `launch()` and, once `wait()` returns, read `h_out`.  `__call__` does the three for host
    tensors.  Build it after the cache is allocated; the graph holds the cache's addresses."""

    def __init__(self, attn: SocketAttention, batch: int):
        cache = attn.kv_cache
        assert cache is not None, "Call setup_cache() first so kv_cache exists"
        dev, dt = cache.k_cache.device, cache.k_cache.dtype
        B, H, Hkv, D = batch, attn.n_head, attn.n_local_heads, attn.head_dim
        assert B == cache.k_cache.shape[0]
        es = torch.empty((), dtype=dt).element_size()
        nq, nkv = B * H * D * es, B * Hkv * D * es
        total = 16 + nq + 2 * nkv
        self.h_in = torch.zeros(total, dtype=torch.uint8).pin_memory()
        self.d_in = torch.zeros(total, dtype=torch.uint8, device=dev)

        def views(buf):
            pos = buf[:8].view(torch.int64)
            q = buf[16:16 + nq].view(dt).view(B, H, D)
            k = buf[16 + nq:16 + nq + nkv].view(dt).view(B, 1, Hkv, D)
            v = buf[16 + nq + nkv:].view(dt).view(B, 1, Hkv, D)
            return pos, q, k, v

        self.h_pos, self.h_q, self.h_k, self.h_v = views(self.h_in)
        d_pos, d_q, d_k, d_v = views(self.d_in)
        self.h_out = torch.empty(B, H, D, dtype=dt).pin_memory()
        self.h2d_bytes, self.d2h_bytes = total, self.h_out.numel() * es
        assert not isinstance(attn.heavy_const, float), "a captured step has a fixed budget"
        self.step = ops.DecodeStep(cache, d_q, d_k, d_v, d_pos, attn.planes, attn.protos_T, self.h_out,
                                   topk=attn.heavy_const, sink=attn.sink_size, window=attn.window_size,
                                   T_max=cache.k_cache.shape[2], temperature=attn.temperature)
        self.done = torch.cuda.Event()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.d_in.copy_(self.h_in, non_blocking=True)
            self.step.run()

    def stage(self, packed: Tensor) -> None:
        """Copy one packed input block (same layout and size as `h_in`, host memory) into the
        staging block."""
        assert packed.numel() * packed.element_size() == self.h_in.numel() and packed.is_contiguous()
        ctypes.memmove(self.h_in.data_ptr(), packed.data_ptr(), self.h_in.numel())

    def launch(self) -> None:
        self.graph.replay()
        self.done.record()

    def wait(self) -> Tensor:
        self.done.synchronize()
        return self.h_out

    @torch.no_grad()
    def __call__(self, q: Tensor, k_new: Tensor, v_new: Tensor, pos: int) -> Tensor:
        self.h_q.copy_(q)
        self.h_k.copy_(k_new)
        self.h_v.copy_(v_new)
        self.h_pos[0] = pos
        self.launch()
        return self.wait()
