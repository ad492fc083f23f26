"""Dense (non-causal) fused self-attention forward with key padding by ``lens``.

Drop-in for ``src/self_attention/kernel.py:359-500`` of ``alexdremov/kernels``: operator
``alexdremov_flash_attention::forward`` with its fake implementation, and the public
``self_attention`` function.  The op body calls ``kb_fa_fwd`` of the sm_100a CUDA library;
the dense schedule is the streaming schedule with a single chunk.  Forward only, no LSE,
as in the reference.  There is no CPU or eager fallback.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.nn.functional as F

from .. import _lib


@torch.library.custom_op("alexdremov_flash_attention::forward", mutates_args=(), device_types=("cuda",))
def attention_forward_adapter(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    lens: Optional[torch.Tensor],
    sm_scale: float,
    autotune: bool,
    prescale: bool,
) -> torch.Tensor:
    batch, heads, T, D = q.shape
    # Contract of the reference op body (self_attention/kernel.py:373-380).
    assert D in (16, 32, 64, 128, 256)
    assert D == k.shape[-1] and D == v.shape[-1]
    assert T == k.shape[-2] and T == v.shape[-2]
    assert q.dtype == k.dtype == v.dtype
    assert sm_scale is not None
    assert lens is None or (lens.dtype == torch.int32 and batch == len(lens) and lens.ndim == 1)

    O = torch.empty_like(q, memory_format=torch.contiguous_format)
    if lens is not None and lens.device != q.device:
        lens = lens.to(q.device)
    p = _lib.SaFwdParams()
    p.q, p.k, p.v = _lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v)
    p.o = O.data_ptr()
    p.lse = None
    p.lens = lens.data_ptr() if lens is not None else None
    p.lens_stride = lens.stride(0) if lens is not None else 0
    p.B, p.H, p.T, p.D = batch, heads, T, D
    p.dtype = _lib.dtype_code(q.dtype)
    p.context_size, p.back_contexts = max(T, 1), 0
    p.sm_scale = float(sm_scale)
    p.flags = _lib.KB_FLAG_PRESCALE_QK if prescale else 0
    p.status = _lib.status_words().data_ptr()
    lib = _lib.load()
    with torch.cuda.device(q.device):
        rc = lib.kb_fa_fwd(ctypes.byref(p), torch.cuda.current_stream(q.device).cuda_stream)
    _lib.check(rc, "kb_fa_fwd")
    return O


@torch.library.register_fake("alexdremov_flash_attention::forward")
def attention_forward_adapter_abstract(q, k, v, lens, sm_scale, autotune, prescale):
    return torch.empty_like(q, memory_format=torch.contiguous_format)


def _padding_masks(T, lens, device):
    if lens is None:
        return None, 1
    valid = (torch.arange(T, device=device).unsqueeze(0) < lens.unsqueeze(-1)).unsqueeze(-1)
    return (valid & valid.transpose(-1, -2)).unsqueeze(1), valid.unsqueeze(1)


def self_attention_reference(q, k, v, lens):
    """Dense SDPA with the key-padding mask, padded rows zeroed; returns ``(out, res_mask)``.

    Checking aid with the reference helper's interface (self_attention/kernel.py:430-449).
    """
    attn_mask, res_mask = _padding_masks(q.shape[-2], lens, q.device)
    return F.scaled_dot_product_attention(query=q, key=k, value=v, attn_mask=attn_mask) * res_mask, res_mask


def self_attention_reference_naive(q, k, v, lens):
    """Explicit-softmax form of :func:`self_attention_reference` (self_attention/kernel.py:452-477)."""
    D = q.shape[-1]
    attn_mask, res_mask = _padding_masks(q.shape[-2], lens, q.device)
    scores = (q / (D**0.5)) @ k.transpose(-1, -2)
    if attn_mask is not None:
        scores = torch.where(attn_mask, scores, -float("inf"))
    result = F.softmax(scores, dim=-1) @ v
    if isinstance(res_mask, int):
        return result, res_mask
    return torch.where(res_mask, result, 0), res_mask


def self_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    lens: Optional[torch.Tensor],
    sm_scale: Optional[float] = None,
    autotune=True,
    prescale=False,
):
    """Non-causal attention over ``(batch, heads, time, head_dim)`` with optional int32 ``lens``.

    Keys at positions ``>= lens[b]`` are ignored and output rows there are 0.  ``autotune`` and
    ``prescale`` are accepted for compatibility and have no effect (fixed sm_100a tile table;
    fp32 scaling).  Interface of ``self_attention`` in the reference (kernel.py:480-500).
    """
    if sm_scale is None:
        sm_scale = q.size(-1) ** -0.5
    return torch.ops.alexdremov_flash_attention.forward(q, k, v, lens, sm_scale, autotune, prescale)
