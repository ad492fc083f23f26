"""The projections on either side of the streaming-attention operator, fused with its layout.

The reference's operator takes ``q, k, v`` as ``[B, H, T, D]`` and returns ``O`` in the same layout
(``src/streaming_attention/kernel.py:1599-1652``); its callers produce them with ``torch.nn.Linear``, a
reshape / transpose and a rotary-embedding pass, and feed ``O`` through another transpose into the
output ``Linear``.  Here the two projections are tcgen05 GEMMs of the C-ABI library that write and read
that layout directly:

* :func:`qkv_rope_projection`: ``x [B, T, E]`` times the stacked weight ``[(H + 2 H_kv) D, E]`` gives
  ``q [B, H, T, D]``, ``k``, ``v [B, H_kv, T, D]`` with the rotary embedding of ``q`` and ``k`` applied to
  the fp32 accumulator (``kb_qkv_rope_proj``);
* :func:`output_projection`: ``o [B, H, T, D]`` times ``w [E_out, H D]`` gives ``y [B, T, E_out]``
  (``kb_out_proj``).

Forward only (no autograd): they serve inference and the forward of a training step.  There is no other
path: shapes the kernels do not take raise.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _lib


def rope_tables(T: int, D: int, base: float = 10000.0, device=None, positions: Optional[torch.Tensor] = None):
    """``(cos, sin)`` as fp32 ``[D / 2, T]``: entry ``[i, t]`` is the cosine / sine of ``positions[t] *
    base ** (-2 i / D)`` (``positions`` defaults to ``0 .. T - 1``).  Frequency-major, the layout the
    kernel's epilogue reads with coalesced loads."""
    pos = torch.arange(T, dtype=torch.float64, device=device) if positions is None else positions.to(torch.float64)
    inv_freq = base ** (-torch.arange(0, D, 2, dtype=torch.float64, device=pos.device) / D)
    ang = inv_freq[:, None] * pos[None, :]
    return ang.cos().float().contiguous(), ang.sin().float().contiguous()


def qkv_rope_projection(x: torch.Tensor, w_qkv: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                        cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None):
    """``q [B, H, T, D], k, v [B, H_kv, T, D] = split(x @ w_qkv.T)`` with rotary embedding on ``q`` and ``k``.

    ``x``: ``[B, T, E]`` fp16 / bf16; ``w_qkv``: ``[(H + 2 H_kv) D, E]`` (query heads, then key heads, then
    value heads); ``cos`` / ``sin``: :func:`rope_tables` output, or both ``None`` for no rotation.
    """
    if not x.is_cuda:
        raise RuntimeError("qkv_rope_projection: CUDA tensors required (there is no CPU path)")
    B, T, E = x.shape
    assert w_qkv.shape == ((heads + 2 * kv_heads) * head_dim, E) and w_qkv.dtype == x.dtype
    assert (cos is None) == (sin is None)
    x, w_qkv = x.contiguous(), w_qkv.contiguous()
    if cos is not None:
        assert cos.shape == (head_dim // 2, T) and sin.shape == cos.shape
        assert cos.dtype == torch.float32 and sin.dtype == torch.float32
        cos, sin = cos.contiguous(), sin.contiguous()
    q = torch.empty((B, heads, T, head_dim), dtype=x.dtype, device=x.device)
    k = torch.empty((B, kv_heads, T, head_dim), dtype=x.dtype, device=x.device)
    v = torch.empty_like(k)
    p = _lib.QkvProjParams()
    p.x, p.w, p.q, p.k, p.v = x.data_ptr(), w_qkv.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr()
    p.rope_cos = cos.data_ptr() if cos is not None else None
    p.rope_sin = sin.data_ptr() if sin is not None else None
    p.B, p.T, p.E, p.H, p.H_kv, p.D = B, T, E, heads, kv_heads, head_dim
    p.dtype = _lib.dtype_code(x.dtype)
    p.status = _lib.status_words().data_ptr()
    with torch.cuda.device(x.device):
        rc = _lib.load().kb_qkv_rope_proj(ctypes.byref(p), torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(rc, "kb_qkv_rope_proj")
    return q, k, v


def output_projection(o: torch.Tensor, w_o: torch.Tensor) -> torch.Tensor:
    """``y [B, T, E_out] = concat_heads(o) @ w_o.T`` for ``o [B, H, T, D]`` (any strides with unit stride
    along ``D``) and ``w_o [E_out, H D]``."""
    if not o.is_cuda:
        raise RuntimeError("output_projection: CUDA tensors required (there is no CPU path)")
    B, H, T, D = o.shape
    assert w_o.ndim == 2 and w_o.shape[1] == H * D and w_o.dtype == o.dtype
    if o.stride(-1) != 1:
        o = o.contiguous()
    w_o = w_o.contiguous()
    y = torch.empty((B, T, w_o.shape[0]), dtype=o.dtype, device=o.device)
    p = _lib.OutProjParams()
    p.o, p.w, p.y = _lib.tensor4(o), w_o.data_ptr(), y.data_ptr()
    p.B, p.T, p.H, p.D, p.E_out = B, T, H, D, w_o.shape[0]
    p.dtype = _lib.dtype_code(o.dtype)
    p.status = _lib.status_words().data_ptr()
    with torch.cuda.device(o.device):
        rc = _lib.load().kb_out_proj(ctypes.byref(p), torch.cuda.current_stream(o.device).cuda_stream)
    _lib.check(rc, "kb_out_proj")
    return y
