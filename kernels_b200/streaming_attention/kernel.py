"""Streaming (chunked block-sparse) attention: Python API, ``torch.library`` operators, autograd.

Drop-in for the operator layer of ``alexdremov/kernels``
(``src/streaming_attention/kernel.py:1270-1652``): same operator names
(``alexdremov_streaming_attention::forward`` / ``::backward``), same argument names and order,
fake (meta) implementations so ``torch.compile`` traces through, the same autograd wiring
and the same public function ``streaming_attention``.  Only the op bodies differ: they call
the sm_100a CUDA library through its C ABI (``include/kernels_b200.h``) instead of
launching Triton kernels.  There is no CPU or eager fallback.

Time is cut into chunks of ``context_size`` tokens; a query attends to every key of its own
chunk and of the ``back_contexts`` chunks before it, and only to positions ``< lens[b]``.
"""

from __future__ import annotations

import ctypes
import logging
from typing import Optional

import torch
import torch.nn.functional as F

from .. import _lib

logger = logging.getLogger(__name__)

_SUPPORTED_HEAD_DIMS = (16, 32, 64, 128, 256)
# Largest dS scratch the backward op will allocate for the single-evaluation kernels.
_MAX_DS_SCRATCH_BYTES = 48 << 30


_device_total_bytes: dict = {}
_ds_scratch: dict = {}


def _ds_scratch_for(device: torch.device, stream_ptr: int, nbytes: int):
    """The dS scratch of the single-evaluation backward: one buffer per (device, stream), kept between
    calls and grown when a larger problem arrives, or ``None`` when the problem's scratch is withheld.

    Whether to provide it is decided from sizes alone (no query of the driver on the hot path): at most
    ``_MAX_DS_SCRATCH_BYTES`` and at most a quarter of the device's total memory.  Calls on one stream run
    one after the other, so they can share a buffer; calls on different streams get their own.
    """
    if nbytes <= 0:
        return None
    idx = device.index if device.index is not None else torch.cuda.current_device()
    total = _device_total_bytes.get(idx)
    if total is None:
        total = _device_total_bytes[idx] = torch.cuda.get_device_properties(idx).total_memory
    if nbytes > _MAX_DS_SCRATCH_BYTES or nbytes > total // 4:
        return None
    key = (idx, stream_ptr)
    buf = _ds_scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        _ds_scratch[key] = None  # let go of the smaller one first
        try:
            buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        except torch.OutOfMemoryError:
            return None  # the two-pass kernels need no such scratch
        _ds_scratch[key] = buf
    return buf


def _flags(prescale_qk: bool, precision: str) -> int:
    if precision not in ("ieee", "tf32"):
        raise RuntimeError(f"precision must be 'ieee' or 'tf32', got {precision!r}")
    f = 0
    if prescale_qk:
        f |= _lib.KB_FLAG_PRESCALE_QK
    if precision == "tf32":
        f |= _lib.KB_FLAG_ALLOW_TF32
    return f


def _check_inputs(q, k, v, lens, context_size, back_contexts, sm_scale):
    # Same contract as the reference op body (kernel.py:1288-1295).
    batch, _, T, D = q.shape
    assert back_contexts >= 0 and context_size >= 1
    assert D in _SUPPORTED_HEAD_DIMS
    assert D == k.shape[-1] and D == v.shape[-1]
    assert T == k.shape[-2] and T == v.shape[-2]
    # the reference wants q.shape[:2] == k.shape[:2] (kernel.py:1291); here k and v may also carry fewer
    # heads that divide the query heads (shared key/value heads): query head h reads head h // (H // H_kv)
    assert k.shape == v.shape and q.shape[0] == k.shape[0]
    assert k.shape[1] >= 1 and q.shape[1] % k.shape[1] == 0
    assert q.dtype == k.dtype == v.dtype
    assert sm_scale is not None
    assert lens is None or (lens.dtype == torch.int32 and batch == len(lens) and lens.ndim == 1)


def _lens_arg(lens: Optional[torch.Tensor], device):
    if lens is None:
        return None, None, 0
    if lens.device != device:
        lens = lens.to(device)
    return lens, lens.data_ptr(), lens.stride(0)


def _clamp_i32(x: int) -> int:
    return int(min(max(int(x), -(2**31)), 2**31 - 1))


@torch.library.custom_op("alexdremov_streaming_attention::forward", mutates_args=(), device_types=("cuda",))
def attention_forward_adapter(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    lens: Optional[torch.Tensor],
    context_size: int,
    back_contexts: int,
    sm_scale: float,
    autotune: bool,
    return_lse: bool,
    prescale_qk: bool,
    precision: str,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Forward op body: allocate ``O`` (and ``LSE``) and launch ``kb_sa_fwd``.

    ``autotune`` is accepted and ignored: tile shapes come from the committed sm_100a table
    (``kb_sa_tile_config``).  ``LSE`` is the base-2 log-sum-exp, or ``torch.empty(0)`` when
    not requested (reference: kernel.py:1297-1300, 1335-1337).
    """
    _check_inputs(q, k, v, lens, context_size, back_contexts, sm_scale)
    B, H, T, D = q.shape
    O = torch.empty_like(q, memory_format=torch.contiguous_format)
    LSE = torch.empty((B, H, T), dtype=torch.float32, device=q.device) if return_lse else None

    lib = _lib.load()
    lens_keep, lens_ptr, lens_stride = _lens_arg(lens, q.device)
    p = _lib.SaFwdParams()
    p.q, p.k, p.v = _lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v)
    p.o = O.data_ptr()
    p.lse = LSE.data_ptr() if LSE is not None else None
    p.lens, p.lens_stride = lens_ptr, lens_stride
    p.B, p.H, p.T, p.D = B, H, T, D
    p.dtype = _lib.dtype_code(q.dtype)
    p.context_size, p.back_contexts = _clamp_i32(context_size), _clamp_i32(back_contexts)
    p.sm_scale = float(sm_scale)
    p.flags = _flags(prescale_qk, precision)
    p.status = _lib.status_words().data_ptr()
    p.H_kv = k.shape[1]
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream(q.device).cuda_stream
        rc = lib.kb_sa_fwd(ctypes.byref(p), stream)
        if rc == _lib.KB_ERR_UNSUPPORTED and k.shape[1] != H:
            # no kernel with shared key/value heads for this dtype / head_dim / layout: repeat the heads
            k_rep, v_rep = (t.repeat_interleave(H // t.shape[1], dim=1) for t in (k, v))
            p.k, p.v, p.H_kv = _lib.tensor4(k_rep), _lib.tensor4(v_rep), H
            rc = lib.kb_sa_fwd(ctypes.byref(p), stream)
    _lib.check(rc, "kb_sa_fwd")
    del lens_keep

    if LSE is None:
        LSE = torch.empty(0)
    return O, LSE


@torch.library.register_fake("alexdremov_streaming_attention::forward")
def attention_forward_adapter_abstract(
    q, k, v, lens, context_size, back_contexts, sm_scale, autotune, return_lse, prescale_qk, precision
):
    out = torch.empty_like(q, memory_format=torch.contiguous_format)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device) if return_lse else torch.empty(0)
    return out, lse


@torch.library.custom_op("alexdremov_streaming_attention::backward", mutates_args=(), device_types=("cuda",))
def attention_backward_adapter(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    lens: Optional[torch.Tensor],
    o: torch.Tensor,
    lse: torch.Tensor,
    do: torch.Tensor,
    context_size: int,
    back_contexts: int,
    sm_scale: float,
    autotune: bool,
    prescale_qk: bool,
    precision: str,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Backward op body: ``(dQ, dK, dV)`` through ``kb_sa_bwd``.

    Scratch is allocated here and handed to the library: ``delta = rowsum(O * dO)`` as
    ``[B, H, T]`` fp32 (reference: kernel.py:1380) and, for the tcgen05 backward that evaluates
    the scores once, room for the 16-bit dS tiles (``kb_sa_bwd_workspace_bytes``; it grows with
    ``(back_contexts + 1) * context_size``; one buffer per device and stream, kept between calls).
    When that room exceeds ``_MAX_DS_SCRATCH_BYTES`` or a quarter of the device's memory, it is
    withheld and the library runs its two-pass kernels, which need none.  ``do`` may arrive in another dtype or with any strides
    (``tests/test_streaming_attention.py:98-112``): it is cast to
    ``q``'s dtype first.
    """
    _check_inputs(q, k, v, lens, context_size, back_contexts, sm_scale)
    B, H, T, D = q.shape
    if do.dtype != q.dtype:
        do = do.to(q.dtype)
    if o.dtype != q.dtype:
        o = o.to(q.dtype)
    if lse.numel() == 0 and q.numel() != 0:
        # The forward was called directly with return_lse=False although a gradient is wanted
        # (the public wrapper never does that): rebuild the log-sum-exp with one more forward.
        _, lse = attention_forward_adapter(
            q.detach(), k.detach(), v.detach(), lens, context_size, back_contexts, sm_scale, autotune, True,
            prescale_qk, precision)
    if lse.dtype != torch.float32 or not lse.is_contiguous():
        lse = lse.to(torch.float32).contiguous()
    assert o.shape == q.shape and do.shape == q.shape and tuple(lse.shape) == (B, H, T)

    DQ = torch.empty_like(q, memory_format=torch.contiguous_format)
    DK = torch.empty_like(k, memory_format=torch.contiguous_format)
    DV = torch.empty_like(v, memory_format=torch.contiguous_format)
    delta = torch.empty((B, H, T), dtype=torch.float32, device=q.device)

    lib = _lib.load()
    ds_ws = None
    if q.numel():
        ws_bytes = int(lib.kb_sa_bwd_workspace_bytes(
            B, H, T, D, _lib.dtype_code(q.dtype), _clamp_i32(context_size), _clamp_i32(back_contexts)))
        ds_ws = _ds_scratch_for(q.device, torch.cuda.current_stream(q.device).cuda_stream, ws_bytes)
    lens_keep, lens_ptr, lens_stride = _lens_arg(lens, q.device)
    p = _lib.SaBwdParams()
    p.q, p.k, p.v, p.o, p.d_o = (_lib.tensor4(t) for t in (q, k, v, o, do))
    p.lse = lse.data_ptr()
    p.dq, p.dk, p.dv = DQ.data_ptr(), DK.data_ptr(), DV.data_ptr()
    p.delta_ws = delta.data_ptr()
    p.ds_ws = ds_ws.data_ptr() if ds_ws is not None else None
    p.ds_ws_bytes = ds_ws.numel() if ds_ws is not None else 0
    p.lens, p.lens_stride = lens_ptr, lens_stride
    p.B, p.H, p.T, p.D = B, H, T, D
    p.dtype = _lib.dtype_code(q.dtype)
    p.context_size, p.back_contexts = _clamp_i32(context_size), _clamp_i32(back_contexts)
    p.sm_scale = float(sm_scale)
    p.flags = _flags(prescale_qk, precision)
    p.status = _lib.status_words().data_ptr()
    p.H_kv = k.shape[1]
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream(q.device).cuda_stream
        rc = lib.kb_sa_bwd(ctypes.byref(p), stream)
        if rc == _lib.KB_ERR_UNSUPPORTED and k.shape[1] != H:
            # no kernel with shared key/value heads for this call: repeat the heads, then add up the
            # gradients of a group's copies
            group = H // k.shape[1]
            k_rep, v_rep = (t.repeat_interleave(group, dim=1) for t in (k, v))
            dk_rep, dv_rep = torch.empty_like(k_rep), torch.empty_like(v_rep)
            p.k, p.v, p.H_kv = _lib.tensor4(k_rep), _lib.tensor4(v_rep), H
            p.dk, p.dv = dk_rep.data_ptr(), dv_rep.data_ptr()
            rc = lib.kb_sa_bwd(ctypes.byref(p), stream)
            if rc == 0:
                DK.copy_(dk_rep.view(B, k.shape[1], group, T, D).float().sum(dim=2))
                DV.copy_(dv_rep.view(B, k.shape[1], group, T, D).float().sum(dim=2))
    _lib.check(rc, "kb_sa_bwd")
    del lens_keep
    return DQ, DK, DV


@torch.library.register_fake("alexdremov_streaming_attention::backward")
def attention_backward_adapter_abstract(
    q, k, v, lens, o, lse, do, context_size, back_contexts, sm_scale, autotune, prescale_qk, precision
):
    return (
        torch.empty_like(q, memory_format=torch.contiguous_format),
        torch.empty_like(k, memory_format=torch.contiguous_format),
        torch.empty_like(v, memory_format=torch.contiguous_format),
    )


def _setup_context(ctx, inputs, output):
    O, LSE = output
    q, k, v, lens, context_size, back_contexts, sm_scale, autotune, _return_lse, prescale_qk, precision = inputs
    ctx.save_for_backward(q, k, v, O, LSE, lens)
    ctx.context_size = context_size
    ctx.back_contexts = back_contexts
    ctx.sm_scale = sm_scale
    ctx.autotune = autotune
    ctx.prescale_qk = prescale_qk
    ctx.precision = precision


def _backward(ctx, do, dlse):
    # Gradients through LSE are not supported (dlse is ignored), as in the reference
    # (kernel.py:1498-1523).
    q, k, v, o, lse, lens = ctx.saved_tensors
    DQ, DK, DV = torch.ops.alexdremov_streaming_attention.backward(
        q=q, k=k, v=v, lens=lens, o=o, lse=lse, do=do,
        context_size=ctx.context_size, back_contexts=ctx.back_contexts, sm_scale=ctx.sm_scale,
        autotune=ctx.autotune, prescale_qk=ctx.prescale_qk, precision=ctx.precision,
    )
    return DQ, DK, DV, None, None, None, None, None, None, None, None


torch.library.register_autograd(
    "alexdremov_streaming_attention::forward", _backward, setup_context=_setup_context
)


def streaming_attention_reference(q, k, v, context_size, back_contexts, lens, scale=None):
    """Dense masked SDPA with the streaming mask, on the tensors' own device.

    Same return triple ``(out, res_mask, sparsity_fraction)`` as the reference helper
    (kernel.py:1533-1563).  O(T^2) memory: a checking aid, never called by the operators.
    """
    T = q.shape[-2]
    dev = q.device
    chunk = torch.div(torch.arange(T, device=dev), context_size, rounding_mode="floor")
    diff = chunk.unsqueeze(1) - chunk.unsqueeze(0)
    attn_mask = (diff >= 0) & (diff <= back_contexts)
    if lens is not None:
        valid = (torch.arange(T, device=dev).unsqueeze(0) < lens.to(dev).unsqueeze(-1)).unsqueeze(-1)
        attn_mask = attn_mask[None, None] & (valid & valid.transpose(-1, -2)).unsqueeze(1)
        res_mask = valid.unsqueeze(1)
    else:
        res_mask = torch.tensor([True], device=dev)
    sparsity_fraction = attn_mask.sum().item() / attn_mask.numel()
    out = F.scaled_dot_product_attention(query=q, key=k, value=v, attn_mask=attn_mask, scale=scale)
    return out, res_mask, sparsity_fraction


@torch.compile(fullgraph=True, dynamic=True)
def _streaming_attention(
    q, k, v, lens, context_size, back_contexts, sm_scale, autotune, return_lse, prescale_qk, precision
):
    requires_grad = any(t.requires_grad for t in (q, k, v))
    O, LSE = torch.ops.alexdremov_streaming_attention.forward(
        q=q, k=k, v=v, lens=lens,
        context_size=context_size, back_contexts=back_contexts, sm_scale=sm_scale,
        autotune=autotune, return_lse=return_lse or requires_grad,
        prescale_qk=prescale_qk, precision=precision,
    )
    if return_lse:
        return O, LSE
    return O


def streaming_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    lens: Optional[torch.Tensor],
    context_size: int,
    back_contexts: int,
    sm_scale: Optional[float] = None,
    autotune=False,
    return_lse=False,
    prescale_qk=False,
    precision="ieee",
):
    """Block-sparse self-attention under a chunked ("streaming") mask, linear in ``time``.

    Args:
        q, k, v: ``(batch, heads, time, head_dim)``; fp32, fp16 or bf16; any strides;
            ``head_dim`` in {16, 32, 64, 128, 256}.  ``k`` and ``v`` may have fewer heads than ``q``
            (a divisor of its head count): consecutive groups of query heads then share a key/value
            head (an extension; the reference requires equal head counts).
        lens: optional int32 ``(batch,)`` sequence lengths; positions ``>= lens[b]`` neither
            attend nor are attended to, and their output rows are 0.
        context_size: chunk length in tokens (>= 1).
        back_contexts: number of earlier chunks a query also sees (>= 0).
        sm_scale: softmax scale, ``head_dim ** -0.5`` by default.
        autotune: accepted for compatibility; the sm_100a tile table is fixed.
        return_lse: also return the base-2 log-sum-exp ``(batch, heads, time)``.
        prescale_qk: accepted for compatibility; scaling is always applied in fp32.
        precision: ``'ieee'`` or ``'tf32'``; fp32 inputs always use IEEE fp32 math.

    Signature and semantics follow ``streaming_attention`` of the reference
    (kernel.py:1599-1652).
    """
    if not torch.compiler.is_compiling():
        for t in (q, k, v):
            torch._dynamo.mark_static(t, 1)
            torch._dynamo.mark_static(t, 3)
    if sm_scale is None:
        sm_scale = q.size(-1) ** -0.5
    return _streaming_attention(
        q=q, k=k, v=v, lens=lens,
        context_size=context_size, back_contexts=back_contexts, sm_scale=sm_scale,
        autotune=autotune, return_lse=return_lse, prescale_qk=prescale_qk, precision=precision,
    )
