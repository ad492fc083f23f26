"""One step of streaming inference: the newest queries against a cache of keys and values.

The reference runs whole sequences only (``src/streaming_attention/kernel.py:1586-1652``); its mask
(``kernel.py:1540-1542``: query ``i`` sees key ``j`` when ``0 <= i // c - j // c <= back``) defines what a
streaming encoder computes when the audio arrives chunk by chunk: the queries of the new chunk attend to
that chunk and to the ``back`` chunks before it.  Here ``k`` and ``v`` hold ``T`` positions (the cache, its
first row on a chunk boundary), ``q`` holds only the LAST ``Tq`` of them, and only those rows are computed:
the result equals rows ``T - Tq ..`` of ``streaming_attention`` over the full tensors, without the work of
the earlier rows.  With a cache of ``back + 1`` chunks and ``Tq = c`` this is the decode step; a larger
``Tq`` is a chunked prefill.

Forward only (inference), through ``kb_sa_fwd`` with ``q_start = T - Tq`` on the tcgen05 kernels
(fp16 / bf16, head_dim 64 or 128).  The other shapes of the operator's surface (fp32, head_dim 16, 32, 256,
odd strides; ``kernel.py:1289``) go through the generic CUDA kernels, which compute whole sequences: the
queries are placed at the end of a zero tensor of ``T`` rows, the whole-sequence operator runs, and the last
``Tq`` rows are returned (correct, at the cost of the earlier rows' work; those shapes are not the
performance path).  There is no CPU path.
"""

import ctypes
import math
from typing import Optional

import torch

from .. import _lib
from .kernel import _clamp_i32, _lens_arg


def streaming_attention_step(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    lens: Optional[torch.Tensor],
    context_size: int,
    back_contexts: int,
    sm_scale: Optional[float] = None,
    return_lse: bool = False,
):
    """``q``: ``[B, H, Tq, D]``, the queries of the last ``Tq`` positions; ``k``, ``v``: ``[B, H_kv, T, D]``
    with ``Tq <= T`` and ``H`` a multiple of ``H_kv``; ``lens``: int32 ``[B]`` valid positions per batch
    element (counted from the first cached row) or None.  Returns ``o`` ``[B, H, Tq, D]`` and, on request,
    the base-2 log-sum-exp ``[B, H, Tq]``.  Rows at positions ``>= len`` come out as zeros."""
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("streaming_attention_step: the tensors must live on a CUDA device (there is no CPU path)")
    assert q.ndim == 4 and k.ndim == 4 and k.shape == v.shape
    B, H, Tq, D = q.shape
    T = k.shape[2]
    assert k.shape[0] == B and k.shape[3] == D and H % k.shape[1] == 0 and q.dtype == k.dtype == v.dtype
    assert 1 <= Tq <= T, "q holds the last Tq of the T cached positions"
    assert context_size >= 1 and back_contexts >= 0
    assert lens is None or (lens.dtype == torch.int32 and lens.ndim == 1 and len(lens) == B)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)

    o = torch.empty((B, H, Tq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, Tq), dtype=torch.float32, device=q.device) if return_lse else None
    lens_keep, lens_ptr, lens_stride = _lens_arg(lens, q.device)
    p = _lib.SaFwdParams()
    p.q, p.k, p.v = _lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v)
    p.o = o.data_ptr()
    p.lse = lse.data_ptr() if lse is not None else None
    p.lens, p.lens_stride = lens_ptr, lens_stride
    p.B, p.H, p.T, p.D = B, H, T, D
    p.dtype = _lib.dtype_code(q.dtype)
    p.context_size, p.back_contexts = _clamp_i32(context_size), _clamp_i32(back_contexts)
    p.sm_scale = float(sm_scale)
    p.flags = 0
    p.status = _lib.status_words().data_ptr()
    p.H_kv = k.shape[1]
    p.q_start = T - Tq
    with torch.cuda.device(q.device):
        rc = _lib.load().kb_sa_fwd(ctypes.byref(p), torch.cuda.current_stream(q.device).cuda_stream)
    del lens_keep
    if rc == _lib.KB_ERR_UNSUPPORTED:
        # no tcgen05 kernel for this dtype / head_dim / layout: whole-sequence call of the generic kernels
        from .kernel import streaming_attention

        with torch.no_grad():
            q_full = torch.zeros((B, H, T, D), dtype=q.dtype, device=q.device)
            q_full[:, :, T - Tq:] = q
            o_full, lse_full = streaming_attention(q_full, k, v, lens, context_size, back_contexts, sm_scale=sm_scale,
                                                   return_lse=True)
        o, lse = o_full[:, :, T - Tq:].contiguous(), lse_full[:, :, T - Tq:].contiguous()
        return (o, lse) if return_lse else o
    _lib.check(rc, "kb_sa_fwd (streaming step)")
    return (o, lse) if return_lse else o
