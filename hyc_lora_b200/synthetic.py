"""Seeded synthetic inputs shaped like the benchmark configurations.

Everything is generated on the CPU in fp32 from one ``torch.Generator`` per
configuration (seed = 1000 + configuration index) and then cast, so a CPU
checker and the GPU path see identical bits.  No dataset item is reproduced:
these tensors only take the shapes and value distributions the configurations
describe.
"""
from __future__ import annotations

import math

import torch


def _gen(config_index: int, salt: int = 0) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(1000 + config_index + 7919 * salt)
    return g


def roundtrip_activation(batch: int = 8, seq: int = 128, hidden: int = 768, planted: int = 8,
                         gain: float = 30.0, dtype=torch.float32, salt: int = 0):
    """Configuration 1: N(0,1) activation with ``planted`` seed-chosen channels
    scaled by ``gain``.  Returns ``(x [B,S,D], planted channel indices)``."""
    g = _gen(1, salt)
    x = torch.randn(batch, seq, hidden, generator=g)
    idx = torch.randperm(hidden, generator=g)[:planted]
    x[..., idx] *= gain
    return x.to(dtype), torch.sort(idx).values


def lora_a_problem(batch: int = 8, seq: int = 128, hidden: int = 768, rank: int = 16, salt: int = 0):
    """Configuration 1's LoRA-A pieces: ``A ~ N(0, 0.02)`` [r, D] and an
    upstream gradient ``G ~ N(0,1)`` [B, S, r] applied at the LoRA-A output."""
    g = _gen(1, 100 + salt)
    a = 0.02 * torch.randn(rank, hidden, generator=g)
    grad = torch.randn(batch, seq, rank, generator=g)
    return a, grad


def sweep_activation(rows: int, hidden: int = 4096, outlier_fraction: float = 0.01,
                     gain: float = 50.0, dtype=torch.bfloat16, salt: int = 0):
    """Configuration 5: Student-t (nu=3) values with a seed-chosen channel set
    of the given fraction scaled by ``gain``.  Returns ``(x [T,D], channels)``.

    A Student-t(3) variate is N(0,1) / sqrt(chi2_3 / 3); it is built from four
    normal draws so that only ``torch.randn`` (stable across devices for a CPU
    generator) is used."""
    g = _gen(5, salt)
    z = torch.randn(rows, hidden, generator=g)
    chi = torch.randn(3, rows, hidden, generator=g).square_().sum(dim=0).div_(3.0).sqrt_()
    x = z.div_(chi)
    k = int(math.ceil(outlier_fraction * hidden - 1e-9))
    idx = torch.randperm(hidden, generator=g)[:k]
    x[:, idx] *= gain
    return x.to(dtype), torch.sort(idx).values


def norm_weight(hidden: int, jitter: float = 0.0, config_index: int = 5, dtype=torch.bfloat16):
    """gamma = 1 (+ jitter * N(0,1))."""
    g = _gen(config_index, 200)
    w = torch.ones(hidden)
    if jitter:
        w = w + jitter * torch.randn(hidden, generator=g)
    return w.to(dtype)


def token_ids(config_index: int, batch: int, seq: int, vocab: int, salt: int = 0):
    g = _gen(config_index, 300 + salt)
    return torch.randint(0, vocab, (batch, seq), generator=g)
