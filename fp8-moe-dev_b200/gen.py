"""Seeded synthetic inputs with the shapes, dtypes, layouts and value distributions of the
layer's benchmark configurations (they stand in for recorded traces, which are not
available offline):

  logits  fp32 N(0,1) [T,256]; bias bf16 N(0,0.1) [256];
  hidden  bf16 N(0,1) [T,7168] quantised per 1x128 block to e4m3, scale = amax/448 stored [56,T];
  weights N(0,0.02) quantised per 128x128 block to e4m3 with fp32 block scales;
  optional Zipf-like skew: logits[:, e] += 1.5 * ln(1 / rank_e), rank_e a fixed permutation of 1..256.

Weights are generated per GLOBAL expert id (seed = base + e), so any sharding of the 256
experts sees identical weights.  With device="cpu" the normal samples come from numpy's
PCG64 generator (bit-identical on every machine); on "cuda" they come from torch's CUDA
generator (fast, used for the large benchmark shapes, not reproducible on a CPU).
"""
from __future__ import annotations

import math
from typing import Tuple

import numpy as np
import torch

H, I, N1, NE, BLK = 7168, 2048, 4096, 256, 128
FP8_MAX = 448.0


class _Normal:
    """Stream of N(0,1) fp32 samples: numpy PCG64 on the CPU, torch's generator on CUDA."""

    def __init__(self, device, seed: int):
        self.device = torch.device(device)
        if self.device.type == "cpu":
            self.rng = np.random.Generator(np.random.PCG64(int(seed)))
        else:
            self.gen = torch.Generator(device=self.device)
            self.gen.manual_seed(int(seed))

    def randn(self, *shape) -> torch.Tensor:
        if self.device.type == "cpu":
            return torch.from_numpy(self.rng.standard_normal(shape, dtype=np.float32))
        return torch.randn(*shape, generator=self.gen, device=self.device, dtype=torch.float32)


def _gen(device, seed: int) -> _Normal:
    return _Normal(device, seed)


def quantize_rows_1x128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [T, K] -> (e4m3 [T, K], scale fp32 [K/128, T])."""
    T, K = x.shape
    xb = x.float().view(T, K // BLK, BLK)
    amax = xb.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (xb / scale.unsqueeze(-1)).clamp_(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(T, K)
    return q, scale.t().contiguous()


def quantize_blocks_128x128(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """w [N, K] -> (e4m3 [N, K], scale fp32 [N/128, K/128])."""
    N, K = w.shape
    wb = w.float().view(N // BLK, BLK, K // BLK, BLK)
    amax = wb.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (wb / scale[:, None, :, None]).clamp_(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(N, K)
    return q, scale.contiguous()


def make_routing(T: int, seed: int = 0, skew: bool = False, device="cpu", skew_seed=None):
    """`skew_seed` fixes WHICH experts are the popular ones (a property of the router, not of a batch);
    it defaults to `seed`.  A second batch for the same router: other `seed`, same `skew_seed`, and the
    first batch's bias."""
    g = _gen(device, seed)
    logits = g.randn(T, NE)
    bias = (0.1 * g.randn(NE)).to(torch.bfloat16)
    if skew:
        perm = np.random.Generator(np.random.PCG64(int(seed if skew_seed is None else skew_seed) + 7919)).permutation(NE)
        rank = torch.from_numpy((perm + 1).astype(np.float32)).to(device)
        logits = logits + 1.5 * torch.log(1.0 / rank)[None, :]
    return logits.contiguous(), bias.contiguous()


def make_hidden(T: int, seed: int = 1, device="cpu", hidden: int = H):
    g = _gen(device, seed)
    x = g.randn(T, hidden).to(torch.bfloat16)
    return quantize_rows_1x128(x)


def make_expert(e_global: int, base_seed: int = 1000, device="cpu", hidden: int = H, inter: int = I):
    """(w1 e4m3 [4096,7168], s1 [32,56], w2 e4m3 [7168,2048], s2 [56,16]) of one global expert; with other
    `hidden` / `inter`: [2*inter, hidden], [2*inter/128, hidden/128], [hidden, inter], [hidden/128, inter/128]."""
    g = _gen(device, base_seed + int(e_global))
    w1 = 0.02 * g.randn(2 * inter, hidden)
    q1, s1 = quantize_blocks_128x128(w1)
    del w1
    w2 = 0.02 * g.randn(hidden, inter)
    q2, s2 = quantize_blocks_128x128(w2)
    return q1, s1, q2, s2


def make_shard(local_expert_offset: int, num_local_experts: int, base_seed: int = 1000, device="cpu",
               out_device=None, hidden: int = H, inter: int = I):
    """Stacked weights of experts [offset, offset + E)."""
    out_device = out_device or device
    E = num_local_experts
    w1 = torch.empty(E, 2 * inter, hidden, dtype=torch.float8_e4m3fn, device=out_device)
    s1 = torch.empty(E, 2 * inter // BLK, hidden // BLK, dtype=torch.float32, device=out_device)
    w2 = torch.empty(E, hidden, inter, dtype=torch.float8_e4m3fn, device=out_device)
    s2 = torch.empty(E, hidden // BLK, inter // BLK, dtype=torch.float32, device=out_device)
    for i in range(E):
        q1, a1, q2, a2 = make_expert(local_expert_offset + i, base_seed, device, hidden, inter)
        w1[i].copy_(q1)
        s1[i].copy_(a1)
        w2[i].copy_(q2)
        s2[i].copy_(a2)
    return w1, s1, w2, s2


def make_experts(expert_ids, base_seed: int = 1000, device="cpu", out_device=None):
    """Stacked weights of the given global experts, in the given order."""
    out_device = out_device or device
    ids = list(expert_ids)
    E = len(ids)
    w1 = torch.empty(E, N1, H, dtype=torch.float8_e4m3fn, device=out_device)
    s1 = torch.empty(E, N1 // BLK, H // BLK, dtype=torch.float32, device=out_device)
    w2 = torch.empty(E, H, I, dtype=torch.float8_e4m3fn, device=out_device)
    s2 = torch.empty(E, H // BLK, I // BLK, dtype=torch.float32, device=out_device)
    for i, e in enumerate(ids):
        q1, a1, q2, a2 = make_expert(e, base_seed, device)
        w1[i].copy_(q1)
        s1[i].copy_(a1)
        w2[i].copy_(q2)
        s2[i].copy_(a2)
    return w1, s1, w2, s2


def expected_rows_per_shard(T: int) -> float:
    """Mean routed rows of a 32-expert shard for uniform routing: 8 T 32 / 256."""
    return 8.0 * T * 32 / NE


def flops_per_row() -> int:
    """2 * (7168*4096 + 2048*7168) = 88,080,384 floating-point operations per routed row."""
    return 2 * (H * N1 + I * H)


def weight_bytes_per_expert() -> int:
    return N1 * H + H * I


__all__ = [
    "make_routing", "make_hidden", "make_expert", "make_shard", "quantize_rows_1x128",
    "quantize_blocks_128x128", "expected_rows_per_shard", "flops_per_row", "weight_bytes_per_expert",
]
_ = math
