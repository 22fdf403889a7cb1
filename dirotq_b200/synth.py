"""Seeded synthetic activations standing in for calibrated DiT activations (which need
non-redistributable checkpoints): N(0,1), plus a planted rank-32 subspace with 20x variance, plus 8
heavy-tailed Student-t(3) channels; bf16."""
import math

import torch


def synth_activations(M: int, D: int, gen: torch.Generator, rank: int = 32, heavy: int = 8) -> torch.Tensor:
    x = torch.randn(M, D, generator=gen)
    rank = min(rank, D)
    v = torch.linalg.qr(torch.randn(D, rank, generator=gen))[0]
    z = torch.randn(M, rank, generator=gen) * math.sqrt(19.0)
    x = x + z @ v.T
    ch = torch.randperm(D, generator=gen)[:heavy]
    num = torch.randn(M, heavy, generator=gen)
    chi = (torch.randn(M, heavy, 3, generator=gen) ** 2).sum(-1) / 3.0
    x[:, ch] = num / chi.sqrt()
    return x.to(torch.bfloat16)
