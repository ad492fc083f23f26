"""GPU: streaming attention forward on e4m3 inputs with per-tile scales (``kb_sa_fwd_fp8``).

The kernel's contract is the streaming attention of the DEQUANTISED q, k, v (what the bytes and the scales
stand for), so the oracle is the CPU restatement of the reference's torch path on the dequantised tensors.
Tolerance row of this entry point: the probabilities are rounded to e4m3 (three mantissa bits) before P V, so
the output is held to max-abs <= 5e-2 and relative L2 <= 4e-2, and the log-sum-exp (formed from the unrounded
probabilities) to 2e-3.  A second comparison, against the 16-bit kernel on the dequantised inputs, checks the
same thing at a size the dense oracle would not finish.
"""

import pytest
import torch

from kernels_b200 import _lib
from oracle import streaming_attention_oracle as SO

pytestmark = pytest.mark.gpu


def _case(B, H, Hk, T, c, back, lens, seed=0, v_spread=1.0):
    from kernels_b200.streaming_attention import dequantize_fp8_tiles, quantize_fp8_tiles, streaming_attention_fp8

    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, T, 128, generator=g)
    k, v = (torch.randn(B, Hk, T, 128, generator=g) for _ in range(2))
    if v_spread != 1.0:  # tiles of very different magnitude: exercises the per-tile v scales
        n = -(-T // 128)
        v = v * torch.logspace(0, math_log10(v_spread), n).repeat_interleave(128)[:T, None]
    q8, qs = quantize_fp8_tiles(q.cuda())
    k8, ks = quantize_fp8_tiles(k.cuda())
    v8, vs = quantize_fp8_tiles(v.cuda())
    lens_t = None if lens is None else torch.tensor(lens, dtype=torch.int32)
    o, lse = streaming_attention_fp8(q8, k8, v8, qs, ks, vs, None if lens_t is None else lens_t.cuda(), c, back,
                                     return_lse=True)
    torch.cuda.synchronize()
    _lib.check_device_status()
    qd, kd, vd = (dequantize_fp8_tiles(a, b).cpu() for a, b in ((q8, qs), (k8, ks), (v8, vs)))
    return o, lse, qd, kd, vd, lens_t


def math_log10(x):
    import math

    return math.log10(x)


@pytest.mark.parametrize("B,H,Hk,T,c,back,lens,v_spread", [
    (2, 2, 2, 640, 128, 2, None, 1.0),
    (2, 4, 2, 700, 48, 3, [700, 333], 1.0),      # shared K/V heads, ragged lengths, chunk edges inside tiles
    (1, 2, 2, 512, 256, 1, [300], 100.0),        # v tiles two orders of magnitude apart
    (1, 2, 1, 130, 10, 5, None, 1.0),
])
def test_fp8_forward_matches_oracle_on_dequantised_inputs(B, H, Hk, T, c, back, lens, v_spread):
    o, lse, qd, kd, vd, lens_t = _case(B, H, Hk, T, c, back, lens, v_spread=v_spread)
    rep = H // Hk
    ref, res_mask, _ = SO.streaming_attention_oracle(qd, kd.repeat_interleave(rep, 1), vd.repeat_interleave(rep, 1), c, back, lens_t)
    mask = torch.ones(B, 1, T, 1, dtype=torch.bool) if lens_t is None else (torch.arange(T)[None] < lens_t[:, None])[:, None, :, None]
    ref = ref * mask
    got = o.float().cpu()
    assert torch.isfinite(got).all()
    assert (got * ~mask).abs().max() == 0  # rows past len are exact zeros
    scale = float(ref.abs().max())
    assert float((got - ref).abs().max()) <= 5e-2 * max(scale, 1.0)
    assert float((got - ref).norm() / ref.norm()) <= 4e-2
    ref_lse = SO.lse_base2_dense(qd, kd.repeat_interleave(rep, 1), c, back, lens_t)
    m = mask[:, 0, :, 0][:, None].expand_as(ref_lse)
    assert float((lse.cpu() - ref_lse)[m].abs().max()) <= 2e-3


def test_fp8_forward_against_the_16_bit_kernel_at_length():
    from kernels_b200.streaming_attention import streaming_attention

    B, H, T, c, back = 1, 4, 4096, 256, 2
    o, lse, qd, kd, vd, _ = _case(B, H, H, T, c, back, None, seed=2)
    ref, ref_lse = streaming_attention(qd.bfloat16().cuda(), kd.bfloat16().cuda(), vd.bfloat16().cuda(), None, c, back,
                                       return_lse=True)
    # the 16-bit kernel rounds the dequantised inputs to bf16 (2^-9 relative) on top of its own P rounding
    assert float((o.float() - ref.float()).norm() / ref.float().norm()) <= 5e-2
    assert float((lse - ref_lse).abs().max()) <= 5e-2


def test_fp8_forward_rejects_what_the_kernel_does_not_take():
    import ctypes

    lib = _lib.load()
    assert lib.kb_sa_fwd_fp8(None, None) == 1
    p = _lib.SaFwdFp8Params()
    p.B, p.H, p.H_kv, p.T, p.D, p.out_dtype, p.context_size = 1, 2, 2, 64, 64, _lib.KB_BF16, 16
    assert lib.kb_sa_fwd_fp8(ctypes.byref(p), None) == _lib.KB_ERR_UNSUPPORTED  # head dim 64
    p.D, p.out_dtype = 128, _lib.KB_F32
    assert lib.kb_sa_fwd_fp8(ctypes.byref(p), None) == _lib.KB_ERR_UNSUPPORTED  # fp32 output
    p.out_dtype, p.H_kv = _lib.KB_BF16, 3
    assert lib.kb_sa_fwd_fp8(ctypes.byref(p), None) == 1
