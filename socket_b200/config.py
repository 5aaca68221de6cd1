"""Static description of a SOCKET sparse-attention layer and the benchmark presets."""
from __future__ import annotations

from dataclasses import dataclass, replace


@dataclass(frozen=True)
class SocketConfig:
    """Knobs of one sparse-attention layer.

    Mirrors the fields the reference spreads over `ModelArgs` (GPT-FAST/model.py:103-118:
    ``L`` tables, ``K`` hyperplanes per table — called ``P`` here —, ``R = 2**P`` buckets,
    ``heavy_const`` = top-k budget) and the ``sink_size`` / ``window_size`` attributes it
    reads with ``getattr(config, ..., 120)`` (model.py:511-512)."""
    batch: int = 1
    n_head: int = 32          # query heads
    n_local_heads: int = 8    # KV heads (the reference's name for them)
    head_dim: int = 128
    context: int = 32768      # T, keys already in the cache
    L: int = 32
    P: int = 8
    temperature: float = 1.0
    topk: int = 1024          # heavy_const
    sink: int = 64
    window: int = 128
    kv_dtype: str = "bf16"    # "bf16" | "f16" | "f32"

    @property
    def R(self) -> int:
        return 1 << self.P

    @property
    def rep(self) -> int:
        return self.n_head // self.n_local_heads

    @property
    def ktot(self) -> int:
        """Length of every row of the sparse list (sink + window + top-k, duplicates kept,
        GPT-FAST/kernels/sparse.py:70-95)."""
        T = self.context
        sink = max(0, min(self.sink, T))
        window = max(0, min(self.window, T))
        n_base = sink + (T - max(T - window, sink) if window > 0 else 0)
        if n_base == 0:
            n_base = 1
        return n_base + min(self.topk, T)

    def kv_bytes(self) -> int:
        return {"bf16": 2, "f16": 2, "f32": 4}[self.kv_dtype]

    def algorithmic_bytes(self) -> int:
        """Bytes one decode step of one layer must move: one uint8 code per key per table
        read once per KV head, plus the K and V rows gathered per query head."""
        a_codes = self.batch * self.n_local_heads * self.context * self.L
        a_kv = self.batch * self.n_head * self.ktot * 2 * self.head_dim * self.kv_bytes()
        return a_codes + a_kv

    def shard_kv_heads(self, world_size: int) -> "SocketConfig":
        """Per-rank view when the KV heads are split over ``world_size`` ranks the way
        GPT-FAST/tp.py:134-137,146-148 divides ``n_head`` and ``n_local_heads``."""
        assert self.n_local_heads % world_size == 0 and self.n_head % world_size == 0
        return replace(self, n_head=self.n_head // world_size,
                       n_local_heads=self.n_local_heads // world_size)


PRESETS = {
    # CPU-runnable op-level case (fp32)
    "c1": SocketConfig(batch=1, context=4096, topk=256, sink=16, window=64, kv_dtype="f32"),
    # op-level, 32K context, bf16 KV
    "c2": SocketConfig(batch=1, context=32768, topk=1024, sink=64, window=128, kv_dtype="bf16"),
    # op-level long context, batch 4, 128K
    "c3": SocketConfig(batch=4, context=131072, topk=2048, sink=64, window=256, kv_dtype="bf16"),
}
