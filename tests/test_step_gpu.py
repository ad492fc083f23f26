"""GPU: the streaming inference step (``kb_sa_fwd`` with ``q_start``), an extension of the reference's operator.

Only the queries of the last ``Tq`` positions are given and computed.  The result must equal the same rows
of the full call: bit for bit when the step's query tiles coincide with the full call's (``q_start`` a
multiple of the 256-row work item), within rounding otherwise (the key tiles of a row are then cut
differently), and within the benchmark contract's tolerance against the CPU oracle.  A rolling cache of
``back + 1`` chunks gives the rows of the whole-sequence call, which is what a streaming encoder relies on.
"""

import pytest
import torch

from kernels_b200 import _lib
from oracle import streaming_attention_oracle as SO

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _fresh_dynamo_cache_per_test():
    # every case calls the compiled whole-sequence entry point with a new (shape, context) combination
    torch._dynamo.reset()
    yield


def _inputs(B, H, Hk, T, D, dtype, seed=5):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, T, D, generator=g).to(dtype)
    k, v = (torch.randn(B, Hk, T, D, generator=g).to(dtype) for _ in range(2))
    return q, k, v


@pytest.mark.parametrize("H,Hk,T,Tq,D,c,back,dtype,lens", [
    (4, 4, 1024, 256, 128, 256, 2, torch.bfloat16, None),        # decode step: one chunk against back + 1 chunks
    (4, 1, 1024, 512, 64, 128, 3, torch.float16, None),          # shared K/V heads
    (2, 2, 1536, 768, 128, 48, 5, torch.bfloat16, [1536, 900]),  # lens inside the computed rows
    (2, 2, 700, 700, 64, 100, 1, torch.float16, [700, 1]),       # q_start = 0: the ordinary call
    (2, 2, 1536, 768, 64, 128, 1, torch.float16, [1000, 100]),   # a batch element that ends before the first query
])
def test_step_equals_full_call_bitwise_on_aligned_starts(H, Hk, T, Tq, D, c, back, dtype, lens):
    from kernels_b200.streaming_attention import streaming_attention, streaming_attention_step

    B = 2
    q, k, v = (t.cuda() for t in _inputs(B, H, Hk, T, D, dtype))
    lens_t = None if lens is None else torch.tensor(lens, dtype=torch.int32).cuda()
    full, lse_full = streaming_attention(q, k, v, lens_t, c, back, return_lse=True)
    n0 = _lib.launch_count()
    out, lse = streaming_attention_step(q[:, :, T - Tq:], k, v, lens_t, c, back, return_lse=True)
    torch.cuda.synchronize()
    assert _lib.launch_count() - n0 == 1
    _lib.check_device_status()
    assert out.shape == (B, H, Tq, D) and lse.shape == (B, H, Tq)
    assert torch.equal(out, full[:, :, T - Tq:])
    valid = torch.ones(B, Tq, dtype=torch.bool, device="cuda") if lens is None else \
        (torch.arange(T - Tq, T, device="cuda")[None] < lens_t[:, None])
    valid = valid[:, None].expand(B, H, Tq)
    assert torch.equal(lse[valid], lse_full[:, :, T - Tq:][valid])


@pytest.mark.parametrize("T,Tq,D,c,back,dtype,lens", [
    (1000, 37, 128, 64, 2, torch.bfloat16, None),
    (777, 500, 64, 10, 7, torch.float16, [777, 600]),
    (640, 1, 128, 128, 4, torch.float16, None),                  # a single new query row
    (515, 258, 64, 256, 0, torch.bfloat16, [515, 300]),
])
def test_step_on_any_start_against_full_call_and_oracle(T, Tq, D, c, back, dtype, lens):
    from kernels_b200.streaming_attention import streaming_attention, streaming_attention_step

    B, H = 2, 3
    q, k, v = _inputs(B, H, H, T, D, dtype, seed=9)
    lens_c = None if lens is None else torch.tensor(lens, dtype=torch.int32)
    lens_t = None if lens is None else lens_c.cuda()
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    full = streaming_attention(qd, kd, vd, lens_t, c, back)
    out, lse = streaming_attention_step(qd[:, :, T - Tq:], kd, vd, lens_t, c, back, return_lse=True)
    torch.cuda.synchronize()
    _lib.check_device_status()
    # same products, key tiles cut at other places: rounding of the 16-bit probabilities only
    assert (out.float() - full[:, :, T - Tq:].float()).abs().max() <= 8e-3
    ref, _, _ = SO.streaming_attention_oracle(q.float(), k.float(), v.float(), c, back, lens_c)
    assert (out.float().cpu() - ref[:, :, T - Tq:]).abs().max() <= 2e-2  # 16-bit kernel against the fp32 oracle
    if lens is not None:
        pad = (torch.arange(T - Tq, T)[None] >= lens_c[:, None])[:, None, :, None].expand(B, H, Tq, D)
        assert (out.cpu()[pad] == 0).all()
    assert torch.isfinite(lse).all()


def test_rolling_cache_reproduces_the_whole_sequence():
    from kernels_b200.streaming_attention import streaming_attention, streaming_attention_step

    B, H, Hk, D, c, back, dtype = 2, 4, 2, 128, 96, 2, torch.bfloat16
    n_chunks = 6
    T = n_chunks * c
    q, k, v = (t.cuda() for t in _inputs(B, H, Hk, T, D, dtype, seed=21))
    full = streaming_attention(q, k, v, None, c, back)
    for n in range(n_chunks):
        first = max(0, n - back) * c  # the cache starts on a chunk boundary
        out = streaming_attention_step(q[:, :, n * c:(n + 1) * c], k[:, :, first:(n + 1) * c], v[:, :, first:(n + 1) * c],
                                       None, c, back)
        assert (out.float() - full[:, :, n * c:(n + 1) * c].float()).abs().max() <= 8e-3, n
    torch.cuda.synchronize()
    _lib.check_device_status()


def test_step_shapes_without_a_tcgen05_kernel_use_the_generic_kernels():
    """fp32 and head dims 16 / 32 / 256 (the rest of the operator's surface): the step equals the whole-sequence
    call's last rows, here against the oracle with the reference's fp32 / fp16 forward tolerances."""
    from kernels_b200.streaming_attention import streaming_attention_step

    for dtype, D, tol in ((torch.float32, 64, 5e-6), (torch.float16, 32, 3e-3), (torch.float32, 256, 5e-6)):
        q, k, v = _inputs(2, 2, 2, 256, D, dtype)
        lens = torch.tensor([256, 200], dtype=torch.int32)
        ref, _, _ = SO.streaming_attention_oracle(q.float(), k.float(), v.float(), 64, 1, lens)
        ref = ref * (torch.arange(256)[None] < lens[:, None])[:, None, :, None]
        out, lse = streaming_attention_step(q[:, :, 128:].cuda(), k.cuda(), v.cuda(), lens.cuda(), 64, 1, return_lse=True)
        assert out.shape == (2, 2, 128, D) and lse.shape == (2, 2, 128)
        assert (out.float().cpu() - ref[:, :, 128:]).abs().max() <= tol, (dtype, D)


def test_step_rejects_bad_shapes():
    from kernels_b200.streaming_attention import streaming_attention_step

    q, k, v = (t.cuda() for t in _inputs(1, 2, 2, 256, 64, torch.float16))
    with pytest.raises(AssertionError):
        streaming_attention_step(torch.cat([q, q], dim=2), k, v, None, 64, 1)  # more queries than positions
