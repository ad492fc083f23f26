"""Streaming attention forward on 8-bit floating-point (e4m3) inputs with per-tile scales.

No counterpart in the reference, whose kernels take fp32, fp16 and bf16
(``src/streaming_attention/kernel.py:1288-1295``); the mask and the result are the reference's
(``kernel.py:1540-1551``), evaluated on the dequantised tensors.  On the tcgen05 tensor cores an e4m3 matmul
instruction covers twice the reduction length of a 16-bit one in the same time, so both matmuls of the
forward need half as many instructions.  ``q``, ``k``, ``v`` come as ``torch.float8_e4m3fn`` tensors with
one fp32 scale per tile of 128 consecutive rows (:func:`quantize_fp8_tiles` produces them); the output is
fp16 or bf16.  Forward only (inference); head_dim 128.  There is no other path: other shapes raise.
"""

from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from .. import _lib
from .kernel import _clamp_i32, _lens_arg

FP8_TILE_ROWS = 128
_E4M3_MAX = 448.0


def quantize_fp8_tiles(x: torch.Tensor):
    """``x [B, H, T, D]`` (any float dtype) -> ``(x8 [B, H, T, D] float8_e4m3fn, scale [B, H, ceil(T/128)] fp32)``
    with ``x ~ x8.float() * scale[tile of the row]``: every tile of 128 rows is scaled so that its largest
    magnitude maps to e4m3's largest value (448)."""
    B, H, T, D = x.shape
    n = -(-T // FP8_TILE_ROWS)
    xf = x.float()
    pad = n * FP8_TILE_ROWS - T
    if pad:
        xf = torch.nn.functional.pad(xf, (0, 0, 0, pad))
    tiles = xf.view(B, H, n, FP8_TILE_ROWS, D)
    scale = (tiles.abs().amax(dim=(-1, -2)) / _E4M3_MAX).clamp_min(1e-12)
    x8 = (tiles / scale[..., None, None]).view(B, H, n * FP8_TILE_ROWS, D)[:, :, :T].to(torch.float8_e4m3fn)
    return x8.contiguous(), scale.contiguous()


def dequantize_fp8_tiles(x8: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """fp32 tensor the 8-bit kernel computes with: ``x8.float() * scale`` of the row's tile."""
    T = x8.shape[2]
    return x8.float() * scale.repeat_interleave(FP8_TILE_ROWS, dim=2)[:, :, :T, None]


def streaming_attention_fp8(
    q8: torch.Tensor, k8: torch.Tensor, v8: torch.Tensor,
    q_scale: torch.Tensor, k_scale: torch.Tensor, v_scale: torch.Tensor,
    lens: Optional[torch.Tensor], context_size: int, back_contexts: int,
    sm_scale: Optional[float] = None, out_dtype: torch.dtype = torch.bfloat16, return_lse: bool = False,
):
    """``q8 [B, H, T, 128]``, ``k8``, ``v8 [B, H_kv, T, 128]`` as ``float8_e4m3fn`` with per-tile scales
    ``[B, heads, ceil(T/128)]``; returns ``o [B, H, T, 128]`` in ``out_dtype`` (and the base-2 log-sum-exp)."""
    if not (q8.is_cuda and k8.is_cuda and v8.is_cuda):
        raise RuntimeError("streaming_attention_fp8: CUDA tensors required (there is no CPU path)")
    assert q8.dtype == k8.dtype == v8.dtype == torch.float8_e4m3fn
    B, H, T, D = q8.shape
    Hk = k8.shape[1]
    assert k8.shape == v8.shape == (B, Hk, T, D) and H % Hk == 0
    n = -(-T // FP8_TILE_ROWS)
    assert q_scale.shape == (B, H, n) and k_scale.shape == v_scale.shape == (B, Hk, n)
    assert context_size >= 1 and back_contexts >= 0
    assert lens is None or (lens.dtype == torch.int32 and lens.ndim == 1 and len(lens) == B)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    q_scale, k_scale, v_scale = (t.float().contiguous() for t in (q_scale, k_scale, v_scale))
    v_max = v_scale.amax(dim=-1).clamp_min(1e-30).contiguous() if n else v_scale.new_ones((B, Hk))
    o = torch.empty((B, H, T, D), dtype=out_dtype, device=q8.device)
    lse = torch.empty((B, H, T), dtype=torch.float32, device=q8.device) if return_lse else None
    lens_keep, lens_ptr, lens_stride = _lens_arg(lens, q8.device)
    p = _lib.SaFwdFp8Params()
    p.q, p.k, p.v = _lib.tensor4(q8), _lib.tensor4(k8), _lib.tensor4(v8)
    p.q_scale, p.k_scale, p.v_scale, p.v_scale_max = (t.data_ptr() for t in (q_scale, k_scale, v_scale, v_max))
    p.o = o.data_ptr()
    p.lse = lse.data_ptr() if lse is not None else None
    p.lens, p.lens_stride = lens_ptr, lens_stride
    p.B, p.H, p.H_kv, p.T, p.D = B, H, Hk, T, D
    p.out_dtype = _lib.dtype_code(out_dtype)
    p.context_size, p.back_contexts = _clamp_i32(context_size), _clamp_i32(back_contexts)
    p.sm_scale = float(sm_scale)
    p.flags = 0
    p.status = _lib.status_words().data_ptr()
    with torch.cuda.device(q8.device):
        rc = _lib.load().kb_sa_fwd_fp8(ctypes.byref(p), torch.cuda.current_stream(q8.device).cuda_stream)
    _lib.check(rc, "kb_sa_fwd_fp8")
    del lens_keep
    return (o, lse) if return_lse else o
