"""CPU oracle for the projections around the attention operator.  TEST INFRASTRUCTURE.

The reference project has no projection code: its operator starts at ``q, k, v [B, H, T, D]``
(``src/streaming_attention/kernel.py:1599-1652``).  What the fused kernels must equal is therefore the
plain composition its callers write: ``torch.nn.functional.linear`` in fp32, a reshape to heads, and the
rotary position embedding in the "rotate half" convention (pairs ``(d, d + D/2)`` of a head), restated
here.  Parity of the kernels is pinned to this restatement only ("parity unpinned" in the sense that the
reference holds no vectors for it).  The product package never imports this module.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def rope_rotate_half(t: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``t``: ``[B, H, T, D]`` fp32; ``cos`` / ``sin``: ``[D/2, T]``.  out[d] = t[d] c - t[d + D/2] s,
    out[d + D/2] = t[d + D/2] c + t[d] s."""
    D = t.shape[-1]
    c, s = cos.t()[None, None], sin.t()[None, None]  # [1, 1, T, D/2]
    lo, hi = t[..., : D // 2], t[..., D // 2:]
    return torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1)


def qkv_rope_projection_oracle(x, w_qkv, heads, kv_heads, head_dim, cos=None, sin=None):
    """fp32 ``(q [B, H, T, D], k [B, H_kv, T, D], v [B, H_kv, T, D])``."""
    B, T, _ = x.shape
    y = F.linear(x.float(), w_qkv.float())  # [B, T, (H + 2 Hk) D]
    nq, nk = heads * head_dim, kv_heads * head_dim
    q = y[..., :nq].reshape(B, T, heads, head_dim).transpose(1, 2)
    k = y[..., nq:nq + nk].reshape(B, T, kv_heads, head_dim).transpose(1, 2)
    v = y[..., nq + nk:].reshape(B, T, kv_heads, head_dim).transpose(1, 2)
    if cos is not None:
        q, k = rope_rotate_half(q, cos.float(), sin.float()), rope_rotate_half(k, cos.float(), sin.float())
    return q.contiguous(), k.contiguous(), v.contiguous()


def output_projection_oracle(o, w_o):
    """fp32 ``y [B, T, E_out]`` for ``o [B, H, T, D]``."""
    B, H, T, D = o.shape
    return F.linear(o.float().transpose(1, 2).reshape(B, T, H * D), w_o.float())
