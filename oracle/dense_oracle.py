"""CPU oracles for the dense self-attention forward and the row softmax.  TEST INFRASTRUCTURE.

The product package never imports this module.  Reference lines followed (paths inside
the reference project):

* ``self_attention_reference`` ......... ``src/self_attention/kernel.py:430-449``
* ``self_attention_reference_naive`` ... ``src/self_attention/kernel.py:452-477``
* ``softmax_naive`` .................... ``src/softmax/kernel.py:94-98``
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def _padding_masks(T, lens, device):
    if lens is None:
        return None, 1
    key_padding = (torch.arange(T, device=device).unsqueeze(0) < lens.unsqueeze(-1)).unsqueeze(-1)
    both = key_padding & key_padding.transpose(-1, -2)
    return both.unsqueeze(1), key_padding.unsqueeze(1)


def self_attention_oracle(q, k, v, lens, scale=None):
    """Non-causal SDPA with a key-padding mask; rows ``>= len`` zeroed.  Returns ``(out, res_mask)``."""
    attn_mask, res_mask = _padding_masks(q.shape[-2], lens, q.device)
    out = F.scaled_dot_product_attention(query=q, key=k, value=v, attn_mask=attn_mask, scale=scale)
    if attn_mask is not None:
        out = torch.nan_to_num(out)
    return out * res_mask, res_mask


def self_attention_oracle_naive(q, k, v, lens, scale=None):
    """Explicit softmax form of the same computation.  Returns ``(out, res_mask)``."""
    D = q.shape[-1]
    scale = D ** -0.5 if scale is None else scale
    attn_mask, res_mask = _padding_masks(q.shape[-2], lens, q.device)
    s = (q * scale) @ k.transpose(-1, -2)
    if attn_mask is not None:
        s = torch.where(attn_mask, s, -float("inf"))
    out = torch.nan_to_num(F.softmax(s, dim=-1)) @ v
    if isinstance(res_mask, int):
        return out, res_mask
    return torch.where(res_mask, out, 0), res_mask


def softmax_oracle(x: torch.Tensor) -> torch.Tensor:
    """``exp(x - max) / sum`` over the last axis, natural exponent (softmax/kernel.py:94-98)."""
    z = x - x.max(-1, keepdim=True).values
    num = torch.exp(z)
    return num / num.sum(dim=-1, keepdim=True)
