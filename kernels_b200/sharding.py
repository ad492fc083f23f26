"""Spreading a streaming-attention problem over several GPUs: batch x heads sharding.

Every (batch, head) slice of the operator is independent in forward and backward, so the
multi-GPU form is one process per GPU, each running the single-GPU operator on its own
slices; no tensor ever crosses a GPU boundary and no collective sits on the data path.
This module holds only the bookkeeping: which slices a rank owns, balanced by the useful
work of each slice (which depends on ``lens[b]``), plus helpers to cut and re-assemble
tensors.  The reference project has no multi-GPU code; this is the one addition around it.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch


def useful_pairs(seq_len: int, context_size: int, back_contexts: int) -> int:
    """Number of unmasked (query, key) pairs of one sequence: the work one head costs."""
    if seq_len <= 0:
        return 0
    c = int(context_size)
    n_full, rem = divmod(int(seq_len), c)
    total, prefix = 0, [0]
    sizes = [c] * n_full + ([rem] if rem else [])
    for s in sizes:
        prefix.append(prefix[-1] + s)
    for ci, s in enumerate(sizes):
        lo = max(0, ci - int(back_contexts))
        total += s * (prefix[ci + 1] - prefix[lo])
    return total


@dataclass(frozen=True)
class Shard:
    """Slices owned by one rank.  ``mode='heads'``: every batch, heads ``heads``;
    ``mode='units'``: explicit ``(b, h)`` pairs (LPT-packed by work)."""

    rank: int
    world: int
    mode: str
    heads: tuple
    units: tuple
    work: int


def partition(B: int, H: int, world: int, lens: Optional[Sequence[int]] = None, T: int = 0,
              context_size: int = 1, back_contexts: int = 0) -> list[Shard]:
    """Assign the ``B*H`` slices to ``world`` ranks.

    If ``world`` divides ``H`` each rank takes heads ``rank, rank+world, ...`` of every batch:
    all ranks then see the same set of lengths, so the split is exactly balanced whatever
    ``lens`` is.  Otherwise slices are packed longest-processing-time-first by useful pairs.
    """
    if world < 1:
        raise ValueError("world must be >= 1")
    lens_eff = [T] * B if lens is None else [max(0, min(int(x), T)) for x in lens]
    cost = [useful_pairs(L, max(1, min(context_size, max(T, 1))), back_contexts) for L in lens_eff]
    if H % world == 0:
        per_head = sum(cost)
        return [
            Shard(r, world, "heads", tuple(range(r, H, world)),
                  tuple((b, h) for b in range(B) for h in range(r, H, world)), per_head * (H // world))
            for r in range(world)
        ]
    order = sorted(((cost[b], b, h) for b in range(B) for h in range(H)), key=lambda t: (-t[0], t[1], t[2]))
    bins = [[] for _ in range(world)]
    load = [0] * world
    for w, b, h in order:
        r = min(range(world), key=lambda i: (load[i], i))
        bins[r].append((b, h))
        load[r] += w
    return [Shard(r, world, "units", (), tuple(sorted(bins[r])), load[r]) for r in range(world)]


def take_local(x: torch.Tensor, shard: Shard) -> torch.Tensor:
    """Cut a full ``[B, H, ...]`` tensor down to the rank's slices.

    ``heads`` mode returns the strided view ``x[:, rank::world]`` (no copy; the kernels take
    strides).  ``units`` mode gathers into ``[1, n_units, ...]``.
    """
    if shard.mode == "heads":
        return x[:, shard.rank :: shard.world]
    idx_b = torch.tensor([b for b, _ in shard.units], device=x.device)
    idx_h = torch.tensor([h for _, h in shard.units], device=x.device)
    return x[idx_b, idx_h].unsqueeze(0)


def local_lens(lens: Optional[torch.Tensor], shard: Shard) -> Optional[torch.Tensor]:
    """``lens`` as the local operator call needs it (``units`` mode folds batch into heads,
    so each unit becomes its own batch entry of one head)."""
    if lens is None or shard.mode == "heads":
        return lens
    return lens[torch.tensor([b for b, _ in shard.units], device=lens.device)].contiguous()


def put_local(full: torch.Tensor, local: torch.Tensor, shard: Shard) -> None:
    """Inverse of :func:`take_local`: write a rank's result back into the full tensor."""
    if shard.mode == "heads":
        full[:, shard.rank :: shard.world] = local
        return
    for i, (b, h) in enumerate(shard.units):
        full[b, h] = local[0, i] if local.shape[0] == 1 else local[i, 0]


def sharded_streaming_attention(q, k, v, lens, context_size, back_contexts, shard: Shard, **kw):
    """Run the single-GPU operator on this rank's slices of full-size ``q, k, v``.

    Returns the local output (``[B, H/world, T, D]`` in ``heads`` mode, ``[n_units, 1, T, D]`` in
    ``units`` mode).  Gradients flow back into the slices of ``q, k, v`` this rank owns.
    """
    from .streaming_attention import streaming_attention

    if shard.mode == "heads":
        return streaming_attention(take_local(q, shard), take_local(k, shard), take_local(v, shard), lens,
                                   context_size, back_contexts, **kw)
    ql, kl, vl = (take_local(t, shard).transpose(0, 1) for t in (q, k, v))  # [n_units, 1, T, D]
    return streaming_attention(ql, kl, vl, local_lens(lens, shard), context_size, back_contexts, **kw)
