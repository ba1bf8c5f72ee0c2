"""Seeded input generators and small utilities shared by the tests.

The generators restate, in this project's own code, the input families the reference's
correctness scripts use (benchmarks/correctness/example_fused_pairtop2_matrix_suite.py:101-166,
example_kernel_vs_pseudo_current.py:87-108) and the config-0 distribution of the benchmark
spec; none of the reference's code is imported here.
"""
from __future__ import annotations

import numpy as np
import torch


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 numpy array of raw bits."""
    return t.detach().cpu().contiguous().view(torch.uint16).numpy().copy()


def from_bits(b: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(b).copy()).view(torch.bfloat16)


def config0_x(m: int, k: int, seed: int = 0) -> torch.Tensor:
    """N(0,1) with a random 1% of K channels scaled x20, bf16."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    cols = torch.randperm(k, generator=g)[: max(1, k // 100)]
    x[:, cols] *= 20.0
    return x.to(torch.bfloat16)


def config0_gamma(k: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed + 1000)
    return (1.0 + 0.1 * torch.randn(k, generator=g)).to(torch.bfloat16)


def config0_w(n: int, k: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed + 2000)
    return (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16)


def outlier_rich_x(m: int, k: int, seed: int = 0) -> torch.Tensor:
    """Small background, two large values in every group of 4, a few hot channels."""
    g = torch.Generator().manual_seed(seed)
    x = 0.03 * torch.randn(m, k, generator=g)
    x4 = x.view(m, k // 4, 4)
    pos = torch.rand(m, k // 4, 4, generator=g).argsort(dim=-1)
    big0 = (8 + 16 * torch.rand(m, k // 4, generator=g)) * torch.sign(torch.randn(m, k // 4, generator=g))
    big1 = (6 + 14 * torch.rand(m, k // 4, generator=g)) * torch.sign(torch.randn(m, k // 4, generator=g))
    x4.scatter_(-1, pos[..., :1], big0.unsqueeze(-1))
    x4.scatter_(-1, pos[..., 1:2], big1.unsqueeze(-1))
    hot = torch.randperm(k, generator=g)[: max(1, (k * 8) // 100)]
    x[:, hot] *= 10 + 30 * torch.rand(hot.numel(), generator=g)
    return x.to(torch.bfloat16)


def pair_friendly_x(m: int, k: int, seed: int = 0) -> torch.Tensor:
    """Exactly two non-zero adjacent pairs in every 8 values (already pair-wise 4:8 sparse)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.zeros(m, k // 8, 4, 2)
    sel = torch.rand(m, k // 8, 4, generator=g).argsort(dim=-1)[..., :2]
    vals = torch.randn(m, k // 8, 2, 2, generator=g) * 3
    x.scatter_(2, sel.unsqueeze(-1).expand(-1, -1, -1, 2), vals)
    return x.view(m, k).to(torch.bfloat16)


def alternating_pair_x(m: int, k: int) -> torch.Tensor:
    """Pairs 0 and 2 of every 8 hold ones, the rest zeros."""
    x = torch.zeros(m, k // 8, 4, 2)
    x[:, :, 0, :] = 1.0
    x[:, :, 2, :] = 1.0
    return x.view(m, k).to(torch.bfloat16)


def tie_x(m: int, k: int, seed: int = 0) -> torch.Tensor:
    """Values from a tiny set so that pair scores tie often and e2m1 midpoints are hit."""
    g = torch.Generator().manual_seed(seed)
    choices = torch.tensor([0.0, -0.0, 0.25, -0.25, 0.5, 0.75, 1.25, -1.75, 2.5, 3.5, -5.0, 6.0])
    idx = torch.randint(0, choices.numel(), (m, k), generator=g)
    return choices[idx].to(torch.bfloat16)


MATRIX_SUITE = {
    "zeros": lambda m, k: torch.zeros(m, k, dtype=torch.bfloat16),
    "ones": lambda m, k: torch.ones(m, k, dtype=torch.bfloat16),
    "pair_friendly": lambda m, k: pair_friendly_x(m, k, 0),
    "alternating_pair": alternating_pair_x,
    "outlier_rich": lambda m, k: outlier_rich_x(m, k, 0),
    "ties": lambda m, k: tie_x(m, k, 0),
    "config0": lambda m, k: config0_x(m, k, 0),
}


def rel_fro(a: np.ndarray, ref: np.ndarray) -> float:
    a = np.asarray(a, np.float64)
    ref = np.asarray(ref, np.float64)
    d = np.linalg.norm(ref)
    return float(np.linalg.norm(a - ref) / d) if d > 0 else float(np.linalg.norm(a - ref))


def raw_violation_rate(q_dense: np.ndarray) -> float:
    """Fraction of 4-byte chunks of a dense sparse payload with more than 2 non-zero bytes."""
    c = q_dense.reshape(q_dense.shape[0], -1, 4)
    return float(((c != 0).sum(axis=-1) > 2).mean())
