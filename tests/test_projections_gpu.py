"""GPU: the fused projections around the attention operator against the CPU oracle.

``kb_qkv_rope_proj`` (x -> q, k, v with rotary embedding, in the attention layout) and ``kb_out_proj``
(o -> y) are tcgen05 GEMMs with no counterpart in the reference; the oracle is the composition its callers
write (fp32 linear + reshape + rotate-half RoPE, ``oracle/projection_oracle.py``).  Tolerance: the 16-bit
kernel against the fp32 oracle, relative L2 <= 1e-2 per tensor and max-abs <= 2e-2 x the tensor's RMS x 8
(one 16-bit rounding of an fp32-accumulated sum), as for the attention gradients.
"""

import ctypes

import pytest
import torch

from kernels_b200 import _lib
from oracle import projection_oracle as PO

pytestmark = pytest.mark.gpu


def _close(name, got, ref):
    got, ref = got.float().cpu(), ref.float()
    assert torch.isfinite(got).all(), name
    rel = float((got - ref).norm() / ref.norm())
    assert rel <= 1e-2, f"{name}: relative L2 {rel:.3e}"
    rms = float(ref.pow(2).mean().sqrt())
    assert float((got - ref).abs().max()) <= 2e-2 * 8 * rms, name


@pytest.mark.parametrize("B,T,E,H,Hk,D,dtype,rope", [
    (2, 300, 256, 4, 2, 128, torch.bfloat16, True),     # partial last token tile, shared K/V heads
    (1, 128, 64, 2, 2, 128, torch.float16, True),       # a single reduction step
    (2, 200, 192, 8, 4, 64, torch.bfloat16, True),      # four heads per feature tile
    (1, 513, 320, 4, 4, 64, torch.float16, False),      # no rotation
    (3, 1, 128, 2, 2, 128, torch.bfloat16, True),       # one token
    (2, 2048, 512, 8, 4, 128, torch.bfloat16, True),    # more tiles than CTA pairs, more reduction steps than ring stages
])
def test_qkv_rope_projection_matches_oracle(B, T, E, H, Hk, D, dtype, rope):
    from kernels_b200.streaming_attention import qkv_rope_projection, rope_tables

    g = torch.Generator().manual_seed(5)
    x = torch.randn(B, T, E, generator=g).to(dtype)
    w = (torch.randn((H + 2 * Hk) * D, E, generator=g) * E ** -0.5).to(dtype)
    cos, sin = rope_tables(T, D) if rope else (None, None)
    ref = PO.qkv_rope_projection_oracle(x, w, H, Hk, D, cos, sin)
    got = qkv_rope_projection(x.cuda(), w.cuda(), H, Hk, D, None if cos is None else cos.cuda(),
                              None if sin is None else sin.cuda())
    torch.cuda.synchronize()
    _lib.check_device_status()
    for name, a, r in zip("qkv", got, ref):
        assert a.shape == r.shape and a.is_contiguous() and a.dtype == dtype
        _close(name, a, r)


@pytest.mark.parametrize("B,T,H,D,E_out,dtype,strided", [
    (2, 300, 4, 128, 512, torch.bfloat16, False),
    (1, 129, 6, 64, 256, torch.float16, False),
    (2, 256, 2, 128, 256, torch.bfloat16, True),   # o as a [B, T, H, D] buffer viewed as [B, H, T, D]
    (3, 1500, 8, 128, 1024, torch.bfloat16, False),  # more tiles than CTA pairs, a last pair with one tile
])
def test_output_projection_matches_oracle(B, T, H, D, E_out, dtype, strided):
    from kernels_b200.streaming_attention import output_projection

    g = torch.Generator().manual_seed(6)
    o = torch.randn(B, H, T, D, generator=g).to(dtype)
    w = (torch.randn(E_out, H * D, generator=g) * (H * D) ** -0.5).to(dtype)
    od = o.cuda()
    if strided:
        od = o.transpose(1, 2).contiguous().cuda().transpose(1, 2)
        assert not od.is_contiguous()
    y = output_projection(od, w.cuda())
    torch.cuda.synchronize()
    _lib.check_device_status()
    assert y.shape == (B, T, E_out) and y.dtype == dtype
    _close("y", y, PO.output_projection_oracle(o, w))


def test_projections_feed_the_attention_operator():
    """x -> (q, k, v) -> streaming attention -> y, every tensor in the attention layout, against the oracles
    chained in fp32 (shared K/V heads)."""
    from kernels_b200.streaming_attention import output_projection, qkv_rope_projection, rope_tables, streaming_attention
    from oracle import streaming_attention_oracle as SO

    B, T, E, H, Hk, D, c, back = 2, 384, 256, 4, 2, 128, 64, 2
    g = torch.Generator().manual_seed(8)
    x = torch.randn(B, T, E, generator=g).bfloat16()
    wqkv = (torch.randn((H + 2 * Hk) * D, E, generator=g) * E ** -0.5).bfloat16()
    wo = (torch.randn(E, H * D, generator=g) * (H * D) ** -0.5).bfloat16()
    cos, sin = rope_tables(T, D)
    q, k, v = qkv_rope_projection(x.cuda(), wqkv.cuda(), H, Hk, D, cos.cuda(), sin.cuda())
    o = streaming_attention(q, k, v, None, c, back)
    y = output_projection(o, wo.cuda())
    torch.cuda.synchronize()
    _lib.check_device_status()
    rq, rk, rv = PO.qkv_rope_projection_oracle(x, wqkv, H, Hk, D, cos, sin)
    rk, rv = (t.repeat_interleave(H // Hk, dim=1) for t in (rk, rv))
    ro, _, _ = SO.streaming_attention_oracle(rq, rk, rv, c, back, None)
    ry = PO.output_projection_oracle(ro, wo)
    rel = float((y.float().cpu() - ry).norm() / ry.norm())
    assert rel <= 2e-2, f"end to end relative L2 {rel:.3e}"


def test_projections_reject_what_the_kernels_do_not_take():
    lib = _lib.load()
    assert lib.kb_qkv_rope_proj(None, None) == 1 and lib.kb_out_proj(None, None) == 1
    p = _lib.QkvProjParams()
    p.B, p.T, p.E, p.H, p.H_kv, p.D, p.dtype = 1, 8, 64, 3, 3, 128, _lib.KB_BF16  # odd head count: no whole tile
    assert lib.kb_qkv_rope_proj(ctypes.byref(p), None) == _lib.KB_ERR_UNSUPPORTED
    p.H, p.H_kv, p.E = 2, 2, 100  # reduction not a multiple of 64
    assert lib.kb_qkv_rope_proj(ctypes.byref(p), None) == _lib.KB_ERR_UNSUPPORTED
    p.E, p.dtype = 64, _lib.KB_F32
    assert lib.kb_qkv_rope_proj(ctypes.byref(p), None) == _lib.KB_ERR_UNSUPPORTED
    o = _lib.OutProjParams()
    o.B, o.T, o.H, o.D, o.E_out, o.dtype = 1, 8, 2, 128, 100, _lib.KB_BF16
    assert lib.kb_out_proj(ctypes.byref(o), None) == _lib.KB_ERR_UNSUPPORTED
