"""A decoder-only transformer around the sparse-attention decode step: the host-side mirror of
`GPT-FAST/model.py` (`ModelArgs` :103-135, `Transformer` :232-333, `TransformerBlock` :336-352,
`Attention` :355-589, `FeedForward` :592-600, `RMSNorm` :603-614, rotary helpers :617-637) and of
the decode loop of `GPT-FAST/generate.py` (:134-189, :246-370), reduced to what the decode
benchmark needs.

What differs from the reference, on purpose:

* decode attention is one `sk_decode_step` per layer (append + hash, soft hash, score, select,
  attend) on cache-native layouts: no code relayout (`model.py:494-499`), no contiguous copy of the
  live K/V prefix (`:541-542`), no `.item()` synchronisation (`:211-212,228,483`), so a whole token
  - all layers, the final norm, the vocabulary projection and the greedy pick - is ONE CUDA graph;
* prefill runs causal flash attention chunk by chunk against the cache (the reference materialises
  a `T x T` boolean mask, `:276-278`, and calls SDPA with it, `:466-474`) and hashes the prompt's
  keys with the bulk tensor-core path;
* tensor parallelism is built in: a rank constructs only its shard (heads split as
  `GPT-FAST/tp.py:124-137` does) and the sum over ranks after `wo` and after the feed-forward is
  issued explicitly (`tp.py`'s forward hook does not fire on the reference's sparse path).

The GEMMs, norms and the dense baseline attention are torch / library kernels: they surround the
path, they are not it.  `mode="dense"` attends over the whole cache with a split-KV flash decode
and is the full-attention baseline of the tokens/s comparison.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from . import ops, tp
from .attention import KVCache
from .synth import hypercube_protos


def find_multiple(n: int, k: int) -> int:
    return n if n % k == 0 else n + k - (n % k)


@dataclass
class ModelArgs:
    """Same fields as the reference's `ModelArgs` (GPT-FAST/model.py:103-135); `K` is the number of
    hyperplanes per table, `R = 2**K` buckets, `heavy_const` the top-k budget.  `sink_size` and
    `window_size` are attributes the reference reads with `getattr(config, ..., 120)`
    (model.py:511-512)."""
    block_size: int = 300000
    vocab_size: int = 32000
    n_layer: int = 1
    n_head: int = 32
    dim: int = 4096
    intermediate_size: Optional[int] = None
    n_local_heads: int = -1
    head_dim: int = 64
    rope_base: float = 40000
    norm_eps: float = 1e-5
    L: int = 32
    R: int = 256
    K: int = 8
    heavy_const: int = 1024
    sink_size: int = 64
    window_size: int = 128
    temperature: float = 1.0

    def __post_init__(self):
        if self.n_local_heads == -1:
            self.n_local_heads = self.n_head
        if self.intermediate_size is None:
            n_hidden = int(2 * (4 * self.dim) / 3)
            self.intermediate_size = find_multiple(n_hidden, 256)
        self.head_dim = self.dim // self.n_head

    @classmethod
    def from_name(cls, name: str, **over):
        return cls(**{**transformer_configs[name], **over})


transformer_configs = {
    # Llama-3-8B shape (random weights in the benchmark)
    "llama-3-8b": dict(block_size=131072, vocab_size=128256, n_layer=32, n_head=32, n_local_heads=8, dim=4096,
                       intermediate_size=14336, rope_base=500000, heavy_const=1024, sink_size=64, window_size=128),
    # Llama-3-70B shape
    "llama-3-70b": dict(block_size=131072, vocab_size=128256, n_layer=80, n_head=64, n_local_heads=8, dim=8192,
                        intermediate_size=28672, rope_base=500000, heavy_const=2048, sink_size=64, window_size=256),
    # small shapes for tests
    "tiny": dict(block_size=4096, vocab_size=512, n_layer=2, n_head=8, n_local_heads=2, dim=1024,
                 intermediate_size=1536, rope_base=10000, heavy_const=64, sink_size=4, window_size=16),
}


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: Tensor) -> Tensor:
        if x.is_cuda:                                   # one fused library kernel
            return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)
        xf = x.float()
        return (xf * torch.rsqrt(torch.mean(xf * xf, dim=-1, keepdim=True) + self.eps)).type_as(x) * self.weight


def precompute_freqs_cis(seq_len: int, n_elem: int, base: float = 10000, device=None) -> Tensor:
    """[seq_len, n_elem/2, 2] (cos, sin) in bf16, as GPT-FAST/model.py:617-623."""
    freqs = 1.0 / (base ** (torch.arange(0, n_elem, 2, device=device)[: n_elem // 2].float() / n_elem))
    ang = torch.outer(torch.arange(seq_len, device=device).float(), freqs)
    return torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.bfloat16)


def apply_rotary_emb(x: Tensor, freqs_cis: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """x [B,S,H,D], freqs_cis [S,D/2,2]: rotate consecutive pairs in fp32 (GPT-FAST/model.py:626-637)."""
    xs = x.float().reshape(*x.shape[:-1], -1, 2)
    fc = freqs_cis.float().view(1, xs.size(1), 1, xs.size(3), 2)
    y = torch.stack([xs[..., 0] * fc[..., 0] - xs[..., 1] * fc[..., 1],
                     xs[..., 1] * fc[..., 0] + xs[..., 0] * fc[..., 1]], -1).flatten(3)
    if out is None:
        return y.type_as(x)
    out.copy_(y.view(out.shape))
    return out


class FeedForward(nn.Module):
    """SwiGLU feed-forward (GPT-FAST/model.py:592-600).  `w1` and `w3` are the two halves of one
    parameter so that the gate and the up projection are one GEMM."""

    def __init__(self, config: ModelArgs, world: int = 1):
        super().__init__()
        self.inter = config.intermediate_size // world
        self.w13 = nn.Linear(config.dim, 2 * self.inter, bias=False)
        self.w2 = nn.Linear(self.inter, config.dim, bias=False)

    @property
    def w1(self) -> Tensor:
        return self.w13.weight[:self.inter]

    @property
    def w3(self) -> Tensor:
        return self.w13.weight[self.inter:]

    def hidden(self, x: Tensor) -> Tensor:
        a, b = self.w13(x).split(self.inter, dim=-1)
        return F.silu(a) * b

    def forward(self, x: Tensor) -> Tensor:
        return self.w2(self.hidden(x))


class Attention(nn.Module):
    """`wqkv` / `wo` around the SOCKET state (planes, protos_T, the cache with codes and norms).
    Under tensor parallelism the module holds `n_head / world` query heads and
    `n_local_heads / world` KV heads; `wqkv` is the rank's [q | k | v] column block and `wo` the
    matching input columns."""

    def __init__(self, config: ModelArgs, world: int = 1):
        super().__init__()
        assert config.n_head % world == 0 and config.n_local_heads % world == 0
        self.n_head = config.n_head // world
        self.n_local_heads = config.n_local_heads // world
        self.head_dim = config.head_dim
        self.dim = config.dim                       # model width (input of wqkv, output of wo)
        self.local_dim = self.n_head * self.head_dim
        self.kv_size = self.n_local_heads * self.head_dim
        self.wqkv = nn.Linear(config.dim, self.local_dim + 2 * self.kv_size, bias=False)
        self.wo = nn.Linear(self.local_dim, config.dim, bias=False)
        self.L, self.K, self.R = config.L, config.K, config.R
        self.heavy_const, self.sink_size, self.window_size = config.heavy_const, config.sink_size, config.window_size
        self.temperature = config.temperature
        # hash parameters: Gaussian hyperplanes and hypercube-corner prototypes (the benchmark's
        # choice; the reference initialises both with randn * 0.02, model.py:377-378)
        self.register_buffer("planes", torch.randn(self.L, self.K, self.head_dim))
        self.register_buffer("protos_T", hypercube_protos(self.K) if self.R == 1 << self.K
                             else torch.randn(self.K, self.R))
        self.kv_cache: Optional[KVCache] = None
        self._step = None

    # ---- prefill: dense causal attention of a chunk of the prompt against the cache
    def prefill(self, x: Tensor, freqs_cis: Tensor, input_pos: Tensor, start: int) -> Tensor:
        B, S, _ = x.shape
        q, k, v = self.wqkv(x).split([self.local_dim, self.kv_size, self.kv_size], dim=-1)
        q = apply_rotary_emb(q.view(B, S, self.n_head, self.head_dim), freqs_cis)
        k = apply_rotary_emb(k.view(B, S, self.n_local_heads, self.head_dim), freqs_cis)
        v = v.view(B, S, self.n_local_heads, self.head_dim)
        cache = self.kv_cache
        if x.is_cuda:
            cache.append(input_pos, k.contiguous(), v.contiguous(), self.planes.to(k.dtype))
        else:                                           # CPU: dense reference flow only (tests)
            cache.k_cache[:, :, input_pos] = k.transpose(1, 2)
            cache.v_cache[:, :, input_pos] = v.transpose(1, 2)
        end = start + S
        y = _causal_attention(q, cache.k_cache[:, :, :end], cache.v_cache[:, :, :end], start)
        return self.wo(y.reshape(B, S, self.local_dim))

    # ---- decode: one token
    def setup_decode(self, batch: int, pos: Tensor, mode: str) -> None:
        dev, dt = self.wqkv.weight.device, self.wqkv.weight.dtype
        self.q_s = torch.empty(batch, self.n_head, self.head_dim, dtype=dt, device=dev)
        self.k_s = torch.empty(batch, 1, self.n_local_heads, self.head_dim, dtype=dt, device=dev)
        self.v_s = torch.empty(batch, 1, self.n_local_heads, self.head_dim, dtype=dt, device=dev)
        self.o_s = torch.empty(batch, self.n_head, self.head_dim, dtype=dt, device=dev)
        self._step = None
        if mode == "sparse":
            cache = self.kv_cache
            self._step = ops.DecodeStep(cache, self.q_s, self.k_s, self.v_s, pos, self.planes.to(dt),
                                        self.protos_T, self.o_s, topk=self.heavy_const, sink=self.sink_size,
                                        window=self.window_size, T_max=cache.k_cache.shape[2],
                                        temperature=self.temperature)

    def decode(self, x: Tensor, freqs_cis: Tensor, pos: Tensor, seqlens: Optional[Tensor], mode: str,
               rope_table: Optional[Tensor] = None, project: bool = True) -> Tensor:
        """x [B,1,dim]; `pos` [1] int64 (device) is the new token's position; `seqlens` [B] int32 =
        keys already cached (dense mode); `freqs_cis` the position's rotary row (CPU flow),
        `rope_table` the whole table (GPU flow: the row is picked on the device)."""
        B = x.shape[0]
        qkv = self.wqkv(x)
        if x.is_cuda:
            # split + rotary embedding of q and k in one launch, straight into the step's inputs
            ops.rope_split(qkv, rope_table, pos, self.n_head, self.n_local_heads, self.q_s, self.k_s, self.v_s)
        else:
            q, k, v = qkv.split([self.local_dim, self.kv_size, self.kv_size], dim=-1)
            apply_rotary_emb(q.view(B, 1, self.n_head, self.head_dim), freqs_cis, out=self.q_s)
            apply_rotary_emb(k.view(B, 1, self.n_local_heads, self.head_dim), freqs_cis, out=self.k_s)
            self.v_s.copy_(v.view(self.v_s.shape))
        cache = self.kv_cache
        if mode == "sparse":
            self._step.run()
            y = self.o_s
        elif x.is_cuda:
            from flash_attn import flash_attn_with_kvcache       # split-KV dense decode (library kernel)
            y = flash_attn_with_kvcache(self.q_s.view(B, 1, self.n_head, self.head_dim),
                                        cache.k_cache.transpose(1, 2), cache.v_cache.transpose(1, 2),
                                        k=self.k_s, v=self.v_s, cache_seqlens=seqlens, causal=True)
        else:
            p = int(pos.item())
            cache.k_cache[:, :, p] = self.k_s[:, 0]
            cache.v_cache[:, :, p] = self.v_s[:, 0]
            y = _causal_attention(self.q_s.view(B, 1, self.n_head, self.head_dim), cache.k_cache[:, :, :p + 1],
                                  cache.v_cache[:, :, :p + 1], p)
        y = y.reshape(B, 1, self.local_dim)
        return self.wo(y) if project else y       # project=False: the caller fuses `wo` with the rank sum


def _causal_attention(q_bshd: Tensor, k_bhtd: Tensor, v_bhtd: Tensor, start: int) -> Tensor:
    """Queries at positions start.. against keys 0..end, causal; GQA.  Library kernels."""
    B, S, H, D = q_bshd.shape
    if q_bshd.is_cuda:
        try:
            from flash_attn import flash_attn_func
            # bottom-right aligned causal mask: query i sees keys 0 .. start + i
            return flash_attn_func(q_bshd, k_bhtd.transpose(1, 2), v_bhtd.transpose(1, 2), causal=True)
        except ImportError:
            pass
    T = k_bhtd.shape[2]
    rep = H // k_bhtd.shape[1]
    mask = (torch.arange(T, device=q_bshd.device)[None, :] <= (start + torch.arange(S, device=q_bshd.device))[:, None])
    y = F.scaled_dot_product_attention(q_bshd.transpose(1, 2), k_bhtd.repeat_interleave(rep, dim=1),
                                       v_bhtd.repeat_interleave(rep, dim=1), attn_mask=mask)
    return y.transpose(1, 2)


class TransformerBlock(nn.Module):
    def __init__(self, config: ModelArgs, world: int = 1):
        super().__init__()
        self.attention = Attention(config, world)
        self.feed_forward = FeedForward(config, world)
        self.ffn_norm = RMSNorm(config.dim, config.norm_eps)
        self.attention_norm = RMSNorm(config.dim, config.norm_eps)
        self.world = world
        self.fused_sum = None                      # tp.FusedRowParallel shared by the model's blocks (decode, GPU)

    def _sum(self, y: Tensor) -> Tensor:
        return tp.all_reduce_sum(y) if self.world > 1 else y

    def prefill(self, x, freqs_cis, input_pos, start):
        h = x + self._sum(self.attention.prefill(self.attention_norm(x), freqs_cis, input_pos, start))
        return h + self._sum(self.feed_forward(self.ffn_norm(h)))

    def decode(self, x, freqs_cis, pos, seqlens, mode, rope_table=None):
        fused = self.fused_sum
        if fused is not None:
            # one kernel per projection: GEMV over this rank's input columns, partial rows pushed to the
            # peers, rank sum and residual added by the owner of each column block
            y = self.attention.decode(self.attention_norm(x), freqs_cis, pos, seqlens, mode, rope_table, project=False)
            h = fused(y, self.attention.wo.weight, res=x.contiguous())
            return fused(self.feed_forward.hidden(self.ffn_norm(h)), self.feed_forward.w2.weight, res=h)
        h = x + self._sum(self.attention.decode(self.attention_norm(x), freqs_cis, pos, seqlens, mode, rope_table))
        return h + self._sum(self.feed_forward(self.ffn_norm(h)))


class Transformer(nn.Module):
    """`world` / `rank`: tensor-parallel layout; every rank builds its own shard (random
    initialisation draws the FULL matrices from one seed and keeps the rank's block, so that the
    ranks together hold exactly the single-GPU model; see `shard_like_reference`)."""

    def __init__(self, config: ModelArgs, world: int = 1, rank: int = 0):
        super().__init__()
        self.config, self.world, self.rank = config, world, rank
        self.tok_embeddings = nn.Embedding(config.vocab_size, config.dim)
        self.layers = nn.ModuleList(TransformerBlock(config, world) for _ in range(config.n_layer))
        self.norm = RMSNorm(config.dim, eps=config.norm_eps)
        self.output = nn.Linear(config.dim, config.vocab_size, bias=False)
        self.register_buffer("freqs_cis", None, persistent=False)
        self.max_batch_size = self.max_seq_length = -1
        self._graph = None
        self.tp_fused = True                       # decode: fuse wo / w2 with the sum over the ranks (GPU, <= 8 rows)
        self._fused_sum = None

    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02) -> "Transformer":
        """Random weights drawn directly in the parameters' dtype on their device (the benchmark has
        no checkpoint).  Hash planes are shared by all ranks; the projections are independent draws
        per rank (each rank's block of a random matrix is a random matrix)."""
        dev = self.tok_embeddings.weight.device
        g = torch.Generator(device=dev).manual_seed(seed)
        gr = torch.Generator(device=dev).manual_seed(seed * 1000003 + 17 * self.rank + 1)
        for name, p in self.named_parameters():
            if p.dim() == 1:
                p.fill_(1.0)
            else:
                shared = name.startswith("tok_embeddings") or name.startswith("output")
                p.copy_(torch.empty(p.shape, dtype=torch.float32, device=dev).normal_(0, std, generator=g if shared else gr))
        for blk in self.layers:
            blk.attention.planes.copy_(torch.randn(blk.attention.planes.shape, generator=g, device=dev))
        return self

    def setup_caches(self, max_batch_size: int, max_seq_length: int) -> None:
        """Per-layer caches (K, V, bucket codes, value norms) and the rotary table; as
        GPT-FAST/model.py:251-278 minus the T x T mask."""
        if self.max_seq_length >= max_seq_length and self.max_batch_size >= max_batch_size:
            return
        dev, dt = self.tok_embeddings.weight.device, self.tok_embeddings.weight.dtype
        max_seq_length = find_multiple(max_seq_length, 8)
        self.max_seq_length, self.max_batch_size = max_seq_length, max_batch_size
        for b in self.layers:
            a = b.attention
            a.kv_cache = KVCache(max_batch_size, max_seq_length, a.n_local_heads, a.head_dim, L=a.L, R=a.R,
                                 dtype=dt, device=dev)
        self.freqs_cis = precompute_freqs_cis(min(self.config.block_size, max_seq_length), self.config.head_dim,
                                              self.config.rope_base, device=dev)
        self._graph = None

    # ------------------------------------------------------------------------------- prefill
    @torch.no_grad()
    def prefill(self, idx: Tensor, chunk: int = 8192) -> Tensor:
        """idx [B,T] prompt token ids -> logits of the last position [B,vocab].  The prompt is
        processed `chunk` tokens at a time: each chunk's keys are appended to the caches (hashed on
        the tensor cores) and its queries attend causally over everything cached so far."""
        B, T = idx.shape
        assert T <= self.max_seq_length and B <= self.max_batch_size
        x_last = None
        for s0 in range(0, T, chunk):
            s1 = min(T, s0 + chunk)
            pos = torch.arange(s0, s1, device=idx.device)
            x = self.tok_embeddings(idx[:, s0:s1])
            fc = self.freqs_cis[s0:s1]
            for layer in self.layers:
                x = layer.prefill(x, fc, pos, s0)
            x_last = x[:, -1]
        return self.output(self.norm(x_last))

    # ------------------------------------------------------------------------------- decode
    def _decode_body(self, mode: str) -> None:
        x = self.tok_embeddings(self._tok)                      # [B,1,dim]
        fc = None if x.is_cuda else self.freqs_cis[self._pos]   # [1,D/2,2]
        for layer in self.layers:
            x = layer.decode(x, fc, self._pos, self._seqlens, mode, self.freqs_cis)
        logits = self.output(self.norm(x))[:, -1]
        self._tok.copy_(torch.argmax(logits, dim=-1, keepdim=True))
        self._pos.add_(1)
        self._seqlens.add_(1)

    @torch.no_grad()
    def setup_decode(self, batch: int, mode: str = "sparse", use_graph: bool = True) -> None:
        """Allocate the decode-time buffers (current token, position, per-layer q/k/v staging,
        the per-layer fused steps) and, on a GPU, capture one token's work in a CUDA graph."""
        dev = self.tok_embeddings.weight.device
        self._mode = mode
        self._tok = torch.zeros(batch, 1, dtype=torch.long, device=dev)
        self._pos = torch.zeros(1, dtype=torch.long, device=dev)
        self._seqlens = torch.zeros(batch, dtype=torch.int32, device=dev)
        for layer in self.layers:
            layer.attention.setup_decode(batch, self._pos, mode)
        if self.world > 1 and dev.type == "cuda" and self.tp_fused and batch <= 8 and \
                self.tok_embeddings.weight.dtype in (torch.bfloat16, torch.float16) and \
                (self.config.dim + 63) // 64 <= torch.cuda.get_device_properties(dev).multi_processor_count:
            if self._fused_sum is None or self._fused_sum.max_batch < batch:
                self._fused_sum = tp.FusedRowParallel(self.config.dim, max(batch, 1), dev)
            for layer in self.layers:
                layer.fused_sum = self._fused_sum
        else:
            for layer in self.layers:
                layer.fused_sum = None
        self._graph = None
        self._host_pos = 0
        if use_graph and dev.type == "cuda":
            saved = (self._tok.clone(), self._pos.clone(), self._seqlens.clone())
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                # position 0 of every cache is overwritten by this dry run and by the capture;
                # decoding starts only after `start_decode`, which the caller follows with real tokens
                self._decode_body(mode)
                side.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    self._decode_body(mode)
            torch.cuda.current_stream(dev).wait_stream(side)
            self._graph = g
            self._tok.copy_(saved[0]); self._pos.copy_(saved[1]); self._seqlens.copy_(saved[2])

    def release_decode(self) -> None:
        """Drop the captured graph and the per-layer steps.  Under tensor parallelism call this
        before `torch.distributed.destroy_process_group()`: a live CUDA graph that holds NCCL
        kernels keeps the communicator busy and the teardown waits for it."""
        self._graph = None
        for layer in self.layers:
            layer.attention._step = None
            layer.fused_sum = None
        if self.tok_embeddings.weight.is_cuda:
            torch.cuda.synchronize(self.tok_embeddings.weight.device)

    @torch.no_grad()
    def start_decode(self, first_token: Tensor, position: int) -> None:
        """`first_token` [B,1] sits at `position` (= number of tokens already cached)."""
        if position >= self.max_seq_length:
            raise RuntimeError(f"start_decode: position {position} outside the caches (max_seq_length="
                               f"{self.max_seq_length})")
        self._host_pos = position                 # host mirror of the device-side position counter
        self._tok.copy_(first_token)
        self._pos.fill_(position)
        self._seqlens.fill_(position)
        if self._mode == "sparse":
            for layer in self.layers:
                layer.attention.kv_cache.prefill_len.fill_(position)

    @torch.no_grad()
    def decode_one_token(self) -> Tensor:
        """Runs one token through the model (greedy); returns the buffer holding the new token.
        Raises before anything is launched when the caches are full (same situation as the
        reference's `_check_input_pos`, GPT-FAST/model.py:279-289, without its device round trip)."""
        if self._host_pos >= self.max_seq_length:
            raise RuntimeError(f"decode position {self._host_pos} outside the caches (max_seq_length="
                               f"{self.max_seq_length}); call setup_caches with a larger length")
        self._host_pos += 1
        if self._graph is not None:
            self._graph.replay()
        else:
            self._decode_body(self._mode)
        return self._tok


@torch.no_grad()
def generate(model: Transformer, prompt: Tensor, max_new_tokens: int, mode: str = "sparse",
             prefill_chunk: int = 8192, use_graph: bool = True, stream_to_host: bool = False):
    """Greedy generation as GPT-FAST/generate.py:246-370: prefill the prompt, take the first new
    token from the prefill logits, then `max_new_tokens - 1` decode steps.  Returns (tokens
    [B, T + max_new_tokens], stats) with `decode_time_s` measured by CUDA events around the decode
    loop and `decode_only_tokens = B * (max_new_tokens - 1)` (generate.py:362-368).  `prompt` may be
    a host tensor; with `stream_to_host` every new token is copied to pinned host memory and waited
    for before the next step is launched (the end-to-end serving pattern)."""
    dev = model.tok_embeddings.weight.device
    B, T = prompt.shape
    prompt_d = prompt.to(dev, non_blocking=True)
    model.setup_caches(B, T + max_new_tokens + 8)
    cuda = dev.type == "cuda"
    e = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if cuda else None
    # the decode graph's dry run scribbles on cache position 0: capture before the prefill
    model.setup_decode(B, mode, use_graph)
    if cuda:
        e[0].record()
    logits = model.prefill(prompt_d, chunk=prefill_chunk)
    first = torch.argmax(logits, dim=-1, keepdim=True)
    if cuda:
        e[1].record()
    seq = torch.empty(B, T + max_new_tokens, dtype=torch.long, device=dev)
    seq[:, :T] = prompt_d
    seq[:, T] = first[:, 0]
    model.start_decode(first, T)
    host_tok = torch.empty(B, 1, dtype=torch.long).pin_memory() if (cuda and stream_to_host) else None
    if cuda:
        torch.cuda.synchronize(dev)
        e[2].record()
    for i in range(1, max_new_tokens):
        tok = model.decode_one_token()
        seq[:, T + i] = tok[:, 0]
        if host_tok is not None:
            host_tok.copy_(tok, non_blocking=True)
            torch.cuda.current_stream(dev).synchronize()
    stats = {"decode_only_tokens": B * max(0, max_new_tokens - 1)}
    if cuda:
        e[3].record()
        torch.cuda.synchronize(dev)
        stats["prefill_time_s"] = e[0].elapsed_time(e[1]) / 1e3
        stats["decode_time_s"] = e[2].elapsed_time(e[3]) / 1e3
    return seq, stats
