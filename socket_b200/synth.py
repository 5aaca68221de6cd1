"""Seeded synthetic inputs for the SOCKET sparse-attention decode path.

One generator, one draw order, so that the CPU oracle, the committed golden
fixtures, the GPU parity tests and the benchmark all see identical values for a
given (shape, seed).  The distributions follow the benchmark configurations:

* planes   [L, P, D]   ~ N(0, 1)            (hash hyperplanes, `Attention.planes`,
                                             GPT-FAST/model.py:377)
* protos_T [P, 2**P]   = hypercube corners  (`Attention.protos_T`, model.py:378; corner
                                             order = itertools.product so that column r is
                                             the big-endian bit pattern of r, consistent with
                                             `pack_bits`, model.py:403-407)
* q        [B, H, D]   ~ N(0, 1)
* K        [B, Hkv, T, D] = N(0,1) * ch_scale[D], ch_scale = exp(N(0,1))
* planted: per (b, kvh) floor(plant_frac*T) positions (randperm) get
           K[pos] = 0.8 * q_dir + 0.2 * N(0,1), q_dir = q[b, kvh*rep] / ||.||
* V        [B, Hkv, T, D] ~ N(0, 1)

Draw order is fixed: planes, q, ch_scale, K, (per group: randperm, noise), V.
Low-precision configs round q, K, V and planes ONCE to the storage dtype; oracle and
kernels then consume the identical rounded values.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Optional

import torch


def hypercube_protos(P: int, dtype=torch.float32) -> torch.Tensor:
    """[P, 2**P] matrix whose column r is the {-1,+1} pattern of r's bits, MSB first."""
    corners = torch.tensor(list(itertools.product([-1.0, 1.0], repeat=P)), dtype=dtype)
    return corners.t().contiguous()


@dataclass
class DecodeInputs:
    planes: torch.Tensor      # [L, P, D]
    protos_T: torch.Tensor    # [P, R]
    q: torch.Tensor           # [B, H, D]
    k: torch.Tensor           # [B, Hkv, T, D]
    v: torch.Tensor           # [B, Hkv, T, D]
    planted: torch.Tensor     # [B, Hkv, n_plant] int64 positions
    meta: dict = field(default_factory=dict)


def make_decode_inputs(
    B: int, H: int, Hkv: int, T: int, D: int = 128, L: int = 32, P: int = 8,
    seed: int = 1234, dtype: torch.dtype = torch.float32, plant_frac: float = 0.01,
    device: Optional[str] = None,
) -> DecodeInputs:
    """Canonical inputs.  With ``device=None`` (CPU generator) the values are the
    contract used by the golden fixtures; with a CUDA device the same distributions are
    drawn by the device generator (different values; used only for large benchmarks)."""
    assert H % Hkv == 0
    rep = H // Hkv
    dev = torch.device(device) if device is not None else torch.device("cpu")
    g = torch.Generator(device=dev).manual_seed(seed)

    def randn(*shape):
        return torch.randn(*shape, generator=g, device=dev, dtype=torch.float32)

    planes = randn(L, P, D)
    q = randn(B, H, D)
    ch_scale = torch.exp(randn(D))
    k = randn(B, Hkv, T, D) * ch_scale
    n_plant = int(plant_frac * T)
    planted = torch.empty(B, Hkv, n_plant, dtype=torch.int64, device=dev)
    for b in range(B):
        for kvh in range(Hkv):
            pos = torch.randperm(T, generator=g, device=dev)[:n_plant]
            noise = randn(n_plant, D)
            q_dir = q[b, kvh * rep]
            q_dir = q_dir / q_dir.norm()
            k[b, kvh, pos] = 0.8 * q_dir + 0.2 * noise
            planted[b, kvh] = pos
    v = randn(B, Hkv, T, D)
    protos_T = hypercube_protos(P).to(dev)
    if dtype != torch.float32:
        planes, q, k, v = (x.to(dtype) for x in (planes, q, k, v))
    return DecodeInputs(planes, protos_T, q, k, v, planted,
                        dict(B=B, H=H, Hkv=Hkv, T=T, D=D, L=L, P=P, seed=seed,
                             dtype=str(dtype), plant_frac=plant_frac))


def make_step_inputs(B: int, H: int, Hkv: int, D: int, steps: int, seed: int,
                     dtype: torch.dtype, device=None):
    """Fresh (q, k, v) for ``steps`` decode steps: q [steps,B,H,D], k/v [steps,B,1,Hkv,D];
    same distributions as above (keys scaled by a log-normal per-channel scale)."""
    dev = torch.device(device) if device is not None else torch.device("cpu")
    g = torch.Generator(device=dev).manual_seed(seed)
    ch_scale = torch.exp(torch.randn(D, generator=g, device=dev))
    q = torch.randn(steps, B, H, D, generator=g, device=dev)
    k = torch.randn(steps, B, 1, Hkv, D, generator=g, device=dev) * ch_scale
    v = torch.randn(steps, B, 1, Hkv, D, generator=g, device=dev)
    return q.to(dtype), k.to(dtype), v.to(dtype)
