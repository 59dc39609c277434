"""Seeded synthetic inputs for the five benchmark/parity configurations of the path.

The reference benchmarks on synthetic tensors only (bench_fusions.py:241-245 of the reference:
``x~randn``, ``y~randint``, ``A~randn``); the configurations here keep those shapes and add the
value distributions of a language-model head: unit-variance activations, a truncated-normal
weight of std 1/sqrt(H) clipped at 2 sigma, uniformly or Zipf distributed labels, and a fraction of
ignored positions. Everything is generated from fixed seeds, on the requested device.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace

import torch


@dataclass(frozen=True)
class Config:
    name: str
    N: int
    H: int
    V: int
    dtype: torch.dtype
    N_chunk_size: int
    ignore_index: int = -1
    frac_ignored: float = 0.02
    logit_scale: float = 1.0
    z_regularization: float = 0.0
    monitoring: bool = False
    labels: str = "uniform"  # or "zipf" (p_k ~ (k+1)^-1.1)
    seed: int = 0

    @property
    def flops(self) -> float:
        """fwd+bwd work on the reference's scale: three N x H x V contractions."""
        return 6.0 * self.N * self.H * self.V


CONFIGS = {
    # CPU-runnable small case, fp32 (multiplied as TF32 on the GPU)
    "c1_small_fp32": Config("c1_small_fp32", 1024, 256, 4096, torch.float32, 256, frac_ignored=0.05, seed=0),
    # default point of the reference's sweeps, fp16
    "c2_default_fp16": Config("c2_default_fp16", 16384, 2048, 131072, torch.float16, 4096, seed=2),
    # default point, bf16, every option on
    "c3_default_bf16_all": Config("c3_default_bf16_all", 16384, 2048, 131072, torch.bfloat16, 4096, logit_scale=0.5,
                                  z_regularization=1e-4, monitoring=True, seed=3),
    # Llama-3-8B-like LM head
    "c4_llama8b_bf16": Config("c4_llama8b_bf16", 65536, 4096, 131072, torch.bfloat16, 8192, frac_ignored=0.03,
                              labels="zipf", seed=4),
    # large-vocabulary scaling case
    "c5_large_vocab_bf16": Config("c5_large_vocab_bf16", 131072, 8192, 262144, torch.bfloat16, 8192, frac_ignored=0.03,
                                  z_regularization=1e-4, labels="zipf", seed=5),
    # small case for profiler captures: operands larger than L2, about 1 GB on the device
    "profile_small_bf16": Config("profile_small_bf16", 4096, 2048, 32768, torch.bfloat16, 4096, seed=6),
    # the same in fp16 (per-tile slabs: the in-place slab transform runs), and with two chunks (the dW contraction
    # then runs once writing and once accumulating)
    "profile_small_fp16": Config("profile_small_fp16", 4096, 2048, 32768, torch.float16, 4096, seed=6),
    "profile_small_2chunks_bf16": Config("profile_small_2chunks_bf16", 8192, 2048, 32768, torch.bfloat16, 4096, seed=6),
    # long tile grids for profiler captures (32 row tiles per chunk, an x chunk of 128 MiB that cannot stay in L2
    # beside the streamed weight): the shape class of the large-hidden configurations at a vocabulary of 16384
    "profile_wide_bf16": Config("profile_wide_bf16", 8192, 8192, 16384, torch.bfloat16, 8192, seed=6),
    # the headline metric's point: default shape in bf16, options off
    "headline_bf16": Config("headline_bf16", 16384, 2048, 131072, torch.bfloat16, 4096, seed=1),
}


def scaled(cfg: Config, **changes) -> Config:
    """A copy of ``cfg`` with some fields replaced (used for sweeps and reduced parity cases)."""
    return replace(cfg, **changes)


def _generator(device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def make_inputs(cfg: Config, device="cuda", vocab_slice: tuple[int, int] | None = None):
    """Returns (x (N,H), y (N,), W (H,V or the requested column slice)).

    W is generated in row blocks so that no float32 copy of the whole matrix is ever alive; with
    ``vocab_slice=(start, stop)`` only those columns are kept (what one rank of a vocabulary-sharded
    run holds) while the random stream stays the one of the full matrix.
    """
    device = torch.device(device)
    gx, gw, gy = (_generator(device, 1000 * cfg.seed + k) for k in range(3))
    x = torch.empty((cfg.N, cfg.H), dtype=cfg.dtype, device=device)
    rows_per_block = max(1, (1 << 26) // cfg.H)
    for r0 in range(0, cfg.N, rows_per_block):
        r1 = min(cfg.N, r0 + rows_per_block)
        x[r0:r1] = torch.randn((r1 - r0, cfg.H), generator=gx, device=device, dtype=torch.float32).to(cfg.dtype)

    v0, v1 = (0, cfg.V) if vocab_slice is None else vocab_slice
    W = torch.empty((cfg.H, v1 - v0), dtype=cfg.dtype, device=device)
    std = 1.0 / math.sqrt(cfg.H)
    rows_per_block = max(1, (1 << 26) // cfg.V)
    for h0 in range(0, cfg.H, rows_per_block):
        h1 = min(cfg.H, h0 + rows_per_block)
        blk = torch.randn((h1 - h0, cfg.V), generator=gw, device=device, dtype=torch.float32)
        blk.clamp_(-2.0, 2.0).mul_(std)  # normal clipped at 2 sigma
        W[h0:h1] = blk[:, v0:v1].to(cfg.dtype)

    if cfg.labels == "zipf":
        ranks = torch.arange(1, cfg.V + 1, device=device, dtype=torch.float64)
        cdf = torch.cumsum(ranks.pow(-1.1), 0)
        cdf /= cdf[-1].clone()
        u = torch.rand(cfg.N, generator=gy, device=device, dtype=torch.float64)
        y = torch.searchsorted(cdf, u).clamp_(max=cfg.V - 1)
    else:
        y = torch.randint(0, cfg.V, (cfg.N,), generator=gy, device=device)
    if cfg.frac_ignored > 0:
        drop = torch.rand(cfg.N, generator=gy, device=device) < cfg.frac_ignored
        y = torch.where(drop, torch.full_like(y, cfg.ignore_index), y)
    return x, y.to(torch.int64), W
