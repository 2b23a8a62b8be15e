"""Seeded synthetic inputs with the shapes and value distributions of the library's benchmark configurations.

Weights are BF16 N(0, 0.02^2); activations BF16 N(0, 1) with 0.1 % of the channels (seeded) multiplied by 20, the
outlier channels real activations show.  Everything is drawn on the CPU from a seeded `torch.Generator`, so every
process, rank and test sees the same bits.
"""
from __future__ import annotations

import torch


def seeded_weight(n: int, k: int, seed: int, std: float = 0.02) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n, k, generator=g) * std).bfloat16()


def seeded_activations(m: int, k: int, seed: int, outliers: bool = True) -> torch.Tensor:
    """BF16 N(0,1) activations with round(0.001 * K) seeded channels multiplied by 20."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    count = round(0.001 * k) if outliers else 0
    if count:
        idx = torch.randperm(k, generator=g)[:count]
        x[:, idx] *= 20.0
    return x.bfloat16()


def zipf_topk(tokens: int, num_experts: int, top_k: int, seed: int, s: float = 1.1) -> torch.Tensor:
    """Expert choice `[tokens, top_k]` (int64) from softmax routing whose logits are N(0,1) plus a Zipf(s) popularity
    prior over the expert index."""
    logits = torch.randn((tokens, num_experts), generator=torch.Generator().manual_seed(seed))
    logits += torch.log(torch.arange(1, num_experts + 1, dtype=torch.float32) ** -s)
    return torch.topk(torch.softmax(logits, -1), top_k, -1).indices


def dirichlet_rows(total_rows: int, num_experts: int, seed: int, alpha: float = 0.3) -> torch.Tensor:
    """Rows per expert (int64 `[num_experts]`, summing to `total_rows`): a multinomial over Dirichlet(alpha) weights."""
    g = torch.Generator().manual_seed(seed)
    gamma = torch._standard_gamma(torch.full((num_experts,), alpha), generator=g).clamp_min(1e-30)
    choice = torch.multinomial(gamma / gamma.sum(), total_rows, replacement=True, generator=g)
    return torch.bincount(choice, minlength=num_experts)
