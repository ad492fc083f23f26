"""Streaming attention over a packed batch (``cu_seqlens`` layout).

The reference's callers hold padded ``[B, H, T, D]`` batches with ``lens``
(``src/streaming_attention/kernel.py:1586-1652``); padded rows are skipped by its kernels but still
allocated, zero-filled and carried through the surrounding layers.  Here the sequences lie one after the
other along the token axis, ``q`` as ``[total, H, D]`` and ``k`` / ``v`` as ``[total, H_kv, D]``, and
``cu_seqlens[b] : cu_seqlens[b + 1]`` are the rows of sequence ``b``.  The mask is the reference's
(``kernel.py:1540-1542``) applied inside every sequence, with chunks counted from the sequence's first
row, so the result equals the padded call row for row (``tests/test_varlen_gpu.py`` checks it bit for bit).

The work is done by ``kb_sa_fwd_varlen`` / ``kb_sa_bwd_varlen`` of the C-ABI library.  The forward is ONE
launch of the tcgen05 kernel over all sequences and the backward one launch of each of its three kernels
(they read every sequence's first row and length from a device copy of ``cu_seqlens``; the last, partial
tile of a sequence is written row by row so that the next sequence's rows stay untouched; the dS scratch is
indexed by packed key tile).  With ``single_launch=False`` both run once per sequence over strided views of
the packed tensors instead, the backward spread over up to eight streams of the library's own ("lanes", each
with its own scratch).  Outputs are written in place.  There is no other path: dtypes, head dims or layouts
those kernels do not take (fp32, head_dim 16, 32 or 256) run sequence by sequence through the padded
operator and its generic CUDA kernels (see ``streaming_attention_varlen``).
"""

import ctypes
import math
from typing import Optional

import torch

from .. import _lib
from .kernel import _clamp_i32


def _free_bytes(device) -> int:
    """Device memory a new allocation can draw on: free in the driver plus cached by torch."""
    free, _total = torch.cuda.mem_get_info(device)
    return free + torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)


def _check(q, k, v, cu_seqlens, context_size, back_contexts):
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("streaming_attention_varlen: the tensors must live on a CUDA device (there is no CPU path)")
    assert q.ndim == 3 and k.ndim == 3 and v.ndim == 3, "q [total, H, D], k and v [total, H_kv, D]"
    assert k.shape == v.shape and q.shape[0] == k.shape[0] and q.shape[2] == k.shape[2]
    assert q.shape[1] % k.shape[1] == 0 and q.dtype == k.dtype == v.dtype
    assert context_size >= 1 and back_contexts >= 0
    assert cu_seqlens.ndim == 1 and cu_seqlens.dtype == torch.int32 and cu_seqlens.numel() >= 1
    cu = cu_seqlens.cpu().contiguous()  # read on the host: the launches are per sequence
    lens = cu[1:] - cu[:-1]
    assert int(cu[0]) == 0 and int(cu[-1]) == q.shape[0] and (lens >= 0).all(), "cu_seqlens must run from 0 to total"
    return cu, int(lens.max()) if lens.numel() else 0


def _params(q, k, v, cu, context_size, back_contexts, sm_scale):
    p = _lib.SaVarlenParams()
    p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    p.cu_seqlens = cu.data_ptr()
    p.B, p.H, p.H_kv, p.D = cu.numel() - 1, q.shape[1], k.shape[1], q.shape[2]
    p.dtype = _lib.dtype_code(q.dtype)
    p.context_size, p.back_contexts = _clamp_i32(context_size), _clamp_i32(back_contexts)
    p.sm_scale = float(sm_scale)
    p.flags = 0
    p.status = _lib.status_words().data_ptr()
    return p


class _StreamingAttentionVarlen(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, context_size, back_contexts, sm_scale, single_launch):
        cu, max_len = _check(q, k, v, cu_seqlens, context_size, back_contexts)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        total, H, D = q.shape
        o = torch.empty_like(q)
        lse = torch.empty((H, total), dtype=torch.float32, device=q.device)
        p = _params(q, k, v, cu, context_size, back_contexts, sm_scale)
        p.o, p.lse = o.data_ptr(), lse.data_ptr()
        cu_dev = cu.to(q.device) if single_launch else None
        p.cu_seqlens_dev = cu_dev.data_ptr() if single_launch else None
        with torch.cuda.device(q.device):
            rc = _lib.load().kb_sa_fwd_varlen(ctypes.byref(p), torch.cuda.current_stream(q.device).cuda_stream)
        _lib.check(rc, "kb_sa_fwd_varlen")
        ctx.mark_non_differentiable(lse)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.cu, ctx.max_len, ctx.cu_dev = cu, max_len, cu_dev
        ctx.args = (context_size, back_contexts, sm_scale)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, o, lse = ctx.saved_tensors
        context_size, back_contexts, sm_scale = ctx.args
        total, H, D = q.shape
        do = do.to(q.dtype).contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        lib = _lib.load()
        n_seq = ctx.cu.numel() - 1
        code, c_i, b_i = _lib.dtype_code(q.dtype), _clamp_i32(context_size), _clamp_i32(back_contexts)
        if ctx.cu_dev is not None:
            # one launch per kernel over the whole batch: delta per packed row, dS tiles per packed key tile
            lanes = 1
            ws_bytes = int(lib.kb_sa_bwd_varlen_workspace_bytes(n_seq, H, total, max(ctx.max_len, 1), D, code, c_i, b_i))
            delta = torch.empty(H * max(total, 1), dtype=torch.float32, device=q.device)
        else:
            # scratch of the longest sequence, reused from sequence to sequence (the launches of a lane are
            # stream-ordered); with more than a few sequences the launches are spread over lanes that run side
            # by side, each with scratch of its own, as long as that stays a small part of the free memory
            ws_bytes = int(lib.kb_sa_bwd_workspace_bytes(1, H, max(ctx.max_len, 1), D, code, c_i, b_i))
            ws_bytes = (ws_bytes + 255) // 256 * 256
            lanes = 1
            if n_seq >= 4:
                lanes = min(8, n_seq // 2)
                while lanes > 1 and lanes * ws_bytes > _free_bytes(q.device) // 8:
                    lanes -= 1
            delta = torch.empty(lanes * H * max(ctx.max_len, 1), dtype=torch.float32, device=q.device)
        ds_ws = torch.empty(max(lanes * ws_bytes, 256), dtype=torch.uint8, device=q.device)
        p = _params(q, k, v, ctx.cu, context_size, back_contexts, sm_scale)
        p.o, p.lse, p.d_o = o.data_ptr(), lse.data_ptr(), do.data_ptr()
        p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
        p.delta_ws, p.ds_ws, p.ds_ws_bytes, p.lanes = delta.data_ptr(), ds_ws.data_ptr(), lanes * ws_bytes, lanes
        p.cu_seqlens_dev = ctx.cu_dev.data_ptr() if ctx.cu_dev is not None else None
        with torch.cuda.device(q.device):
            rc = lib.kb_sa_bwd_varlen(ctypes.byref(p), torch.cuda.current_stream(q.device).cuda_stream)
        _lib.check(rc, "kb_sa_bwd_varlen")
        return dq, dk, dv, None, None, None, None, None


def streaming_attention_varlen(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens: torch.Tensor,
    context_size: int,
    back_contexts: int,
    sm_scale: Optional[float] = None,
    return_lse: bool = False,
    single_launch: bool = True,
):
    """Streaming attention of every sequence of a packed batch; differentiable in q, k, v.

    ``q``: ``[total, H, D]``; ``k``, ``v``: ``[total, H_kv, D]`` with ``H`` a multiple of ``H_kv``;
    ``cu_seqlens``: int32 ``[B + 1]``, from 0 to ``total``.  Returns ``o`` ``[total, H, D]`` (and the base-2
    log-sum-exp ``[H, total]`` when ``return_lse``).  ``sm_scale`` defaults to ``D ** -0.5`` as in the
    reference (``kernel.py:1622-1623``).  ``single_launch=False`` runs the forward as one launch per sequence
    (the same bits; only worth it for a few long sequences when a device copy of ``cu_seqlens`` is unwanted).
    """
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    if q.is_cuda and (q.dtype == torch.float32 or q.shape[-1] not in (64, 128)) and q.shape[-1] in (16, 32, 64, 128, 256):
        return _varlen_generic(q, k, v, cu_seqlens, context_size, back_contexts, sm_scale, return_lse)
    o, lse = _StreamingAttentionVarlen.apply(q, k, v, cu_seqlens, context_size, back_contexts, sm_scale, single_launch)
    return (o, lse) if return_lse else o


def _varlen_generic(q, k, v, cu_seqlens, context_size, back_contexts, sm_scale, return_lse):
    """Shapes without a tcgen05 kernel (the rest of the operator's surface, ``kernel.py:1289``): every sequence
    goes through the padded operator as a batch of one (generic CUDA kernels, autograd included), and the
    results are concatenated.  Same rows as the packed kernels would give; not a performance path."""
    from .kernel import streaming_attention

    cu, _ = _check(q, k, v, cu_seqlens, context_size, back_contexts)
    outs, lses = [], []
    for b in range(cu.numel() - 1):
        r0, r1 = int(cu[b]), int(cu[b + 1])
        if r1 == r0:
            continue
        qs, ks, vs = (t[r0:r1].transpose(0, 1).unsqueeze(0) for t in (q, k, v))  # [1, heads, len, D] views
        o, lse = streaming_attention(qs, ks, vs, None, context_size, back_contexts, sm_scale=sm_scale, return_lse=True)
        outs.append(o[0].transpose(0, 1))
        lses.append(lse[0])
    if not outs:
        o, lse = torch.empty_like(q), torch.empty((q.shape[1], 0), dtype=torch.float32, device=q.device)
    else:
        o, lse = torch.cat(outs, dim=0), torch.cat(lses, dim=1)
    return (o, lse.detach()) if return_lse else o
