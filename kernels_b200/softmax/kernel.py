"""Row softmax over the last axis.

Drop-in for ``softmax`` of ``alexdremov/kernels`` (``src/softmax/kernel.py:74-91``): flattens to
``[rows, cols]`` and calls ``kb_softmax_fwd`` of the sm_100a CUDA library (one pass over HBM).
There is no CPU or eager fallback.
"""

from __future__ import annotations

import ctypes

import torch

from .. import _lib


def softmax(x: torch.Tensor) -> torch.Tensor:
    """``exp(x - max) / sum(exp(x - max))`` over the last axis; fp32, fp16 or bf16 CUDA tensor."""
    if not x.is_cuda:
        raise RuntimeError("kernels_b200.softmax: CUDA tensor required (there is no CPU path)")
    shape = x.shape
    x2 = x.reshape(-1, shape[-1]) if x.dim() != 2 else x
    if x2.numel() and x2.stride(-1) != 1:
        x2 = x2.contiguous()
    rows, cols = x2.shape
    y = torch.empty((rows, cols), dtype=x.dtype, device=x.device)
    p = _lib.SoftmaxParams()
    p.x, p.y = x2.data_ptr(), y.data_ptr()
    p.rows, p.cols = rows, cols
    p.x_row_stride, p.y_row_stride = x2.stride(0) if rows else cols, cols
    p.dtype = _lib.dtype_code(x.dtype)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        rc = lib.kb_softmax_fwd(ctypes.byref(p), torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(rc, "kb_softmax_fwd")
    return y.view(*shape)


def softmax_naive(x: torch.Tensor) -> torch.Tensor:
    """Plain torch form of the same function (checking aid; softmax/kernel.py:94-98)."""
    z = x - x.max(-1, keepdim=True).values
    num = torch.exp(z)
    return num / num.sum(dim=-1, keepdim=True)
