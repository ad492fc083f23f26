"""Seeded synthetic inputs for the streaming-attention benchmarks and tests.

There is no dataset on this path: the reference benchmarks on random tensors
(``benchmark/benchmark_streaming_attention.py:43-111`` of the reference).  The recipe here
makes the data of a (batch, head) slice independent of how slices are spread over GPUs:
``lens`` comes from one seeded CPU generator, then every slice has its own generator.
"""

from __future__ import annotations

import torch


def make_lens(B: int, lo: int, hi: int, seed: int = 0) -> torch.Tensor:
    """int32 ``[B]`` lengths ~ Uniform-int[lo, hi] from a seeded CPU generator."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(lo, hi + 1, (B,), generator=g, dtype=torch.int32)


def make_slice(b: int, h: int, H: int, T: int, D: int, seed: int = 0, qk_scale: float = 1.0):
    """fp32 ``q, k, v, do`` of shape ``[T, D]`` for one (batch, head) slice.

    The generator is seeded with ``seed * 1_000_003 + b * H + h``; ``q, k, v`` are
    ``N(0, 1) * qk_scale`` and ``do`` is ``N(0, 1)``.
    """
    g = torch.Generator(device="cpu").manual_seed(seed * 1_000_003 + b * H + h)
    q = torch.randn(T, D, generator=g) * qk_scale
    k = torch.randn(T, D, generator=g) * qk_scale
    v = torch.randn(T, D, generator=g) * qk_scale
    do = torch.randn(T, D, generator=g)
    return q, k, v, do
