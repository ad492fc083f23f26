"""GPU: streaming attention over a packed batch (``cu_seqlens``), an extension of the reference's operator.

The packed call must equal the padded call (``streaming_attention`` with ``lens``) row for row and bit for
bit: both run the same tcgen05 kernels over the same tiles of every sequence, the packed one in one launch per
kernel over the whole batch or, with ``single_launch=False``, through strided views of the packed tensors.  The padded call in turn is pinned to the oracle by the other GPU tests; one case
here is also checked against the oracle directly, per sequence, with the benchmark contract's tolerances.
"""

import pytest
import torch

from kernels_b200 import _lib
from oracle import streaming_attention_oracle as SO

pytestmark = pytest.mark.gpu


def _pack(t, lens):
    """[B, H, T, D] padded -> [total, H, D] packed."""
    return torch.cat([t[b, :, :L].transpose(0, 1) for b, L in enumerate(lens)], dim=0).contiguous()


def _cu(lens):
    return torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)


@pytest.mark.parametrize("H,Hk,T,D,c,back,dtype,lens", [
    (4, 4, 700, 128, 48, 3, torch.bfloat16, [700, 333, 1]),
    (8, 2, 520, 64, 128, 1, torch.float16, [130, 520, 0, 257]),   # shared K/V heads, an empty sequence
    (2, 2, 1100, 128, 256, 2, torch.float16, [1100, 1024]),
    (3, 1, 300, 64, 10, 5, torch.bfloat16, [299, 17, 128]),
    (2, 2, 260, 128, 32, 2, torch.float16, [5, 130, 256, 257, 1, 127, 128, 129, 0, 260]),  # every kind of last tile
])
@pytest.mark.parametrize("single_launch", [True, False])
def test_packed_equals_padded_bitwise(H, Hk, T, D, c, back, dtype, lens, single_launch):
    from kernels_b200.streaming_attention import streaming_attention, streaming_attention_varlen

    B = len(lens)
    g = torch.Generator().manual_seed(11)
    q = torch.randn(B, H, T, D, generator=g).to(dtype).cuda()
    k, v = (torch.randn(B, Hk, T, D, generator=g).to(dtype).cuda() for _ in range(2))
    do = torch.randn(B, H, T, D, generator=g).to(dtype).cuda()
    lens_t = torch.tensor(lens, dtype=torch.int32).cuda()
    valid = (torch.arange(T, device="cuda")[None] < lens_t[:, None])[:, None, :, None]
    do = do * valid

    qp, kp, vp = (t.detach().clone().requires_grad_() for t in (q, k, v))
    out_pad, lse_pad = streaming_attention(qp, kp, vp, lens_t, c, back, return_lse=True)
    out_pad.backward(do)

    qs, ks, vs = (_pack(t, lens).requires_grad_() for t in (q, k, v))
    n0 = _lib.launch_count()
    out, lse = streaming_attention_varlen(qs, ks, vs, _cu(lens), c, back, return_lse=True, single_launch=single_launch)
    n1 = _lib.launch_count()
    out.backward(_pack(do, lens))
    torch.cuda.synchronize()
    n2 = _lib.launch_count()
    _lib.check_device_status()
    live = sum(1 for L in lens if L > 0)
    # one launch of each kernel (forward; delta, main, dQ) for the whole batch, or one per sequence
    assert n1 - n0 == (1 if single_launch else live) and n2 - n1 == (3 if single_launch else 3 * live)

    assert out.shape == qs.shape and lse.shape == (H, sum(lens))
    assert torch.equal(out, _pack(out_pad.detach(), lens))
    assert torch.equal(lse, torch.cat([lse_pad[b, :, :L] for b, L in enumerate(lens)], dim=1))
    assert torch.equal(qs.grad, _pack(qp.grad, lens))
    assert torch.equal(ks.grad, _pack(kp.grad, lens))
    assert torch.equal(vs.grad, _pack(vp.grad, lens))


def test_packed_against_oracle_per_sequence():
    from kernels_b200.streaming_attention import streaming_attention_varlen

    H, D, c, back, dtype, lens = 4, 128, 64, 2, torch.bfloat16, [450, 129, 64]
    g = torch.Generator().manual_seed(3)
    total = sum(lens)
    q, k, v, do = (torch.randn(total, H, D, generator=g).to(dtype) for _ in range(4))
    qs, ks, vs = (t.cuda().requires_grad_() for t in (q, k, v))
    out = streaming_attention_varlen(qs, ks, vs, _cu(lens), c, back)
    out.backward(do.cuda())
    torch.cuda.synchronize()
    _lib.check_device_status()
    r0 = 0
    for L in lens:
        sl = slice(r0, r0 + L)
        qf, kf, vf = (t[sl].transpose(0, 1)[None].float().clone().requires_grad_() for t in (q, k, v))
        ref, _, _ = SO.streaming_attention_oracle(qf, kf, vf, c, back, None)
        ref.backward(do[sl].transpose(0, 1)[None].float())
        got = out[sl].detach().cpu().float().transpose(0, 1)[None]
        assert (got - ref.detach()).abs().max() <= 2e-2  # fp16 / bf16 kernel against the fp32 oracle
        for name, gpu_grad, ref_grad in (("dq", qs.grad, qf.grad), ("dk", ks.grad, kf.grad), ("dv", vs.grad, vf.grad)):
            gg = gpu_grad[sl].cpu().float().transpose(0, 1)[None]
            assert float((gg - ref_grad).norm() / ref_grad.norm()) <= 2e-2, name
        r0 += L


def test_packed_shapes_without_a_tcgen05_kernel_use_the_generic_kernels():
    """fp32 and head dim 32: sequence by sequence through the padded operator (generic CUDA kernels), forward and
    backward, against the oracle per sequence."""
    from kernels_b200.streaming_attention import streaming_attention_varlen

    for dtype, D, tol_o, tol_g in ((torch.float32, 64, 5e-6, 5e-5), (torch.float16, 32, 3e-3, 1e-2)):
        H, c, back, lens = 2, 16, 2, [100, 0, 37]
        g = torch.Generator().manual_seed(4)
        total = sum(lens)
        q, k, v, do = (torch.randn(total, H, D, generator=g).to(dtype) for _ in range(4))
        qs, ks, vs = (t.cuda().requires_grad_() for t in (q, k, v))
        out, lse = streaming_attention_varlen(qs, ks, vs, _cu(lens), c, back, return_lse=True)
        out.backward(do.cuda())
        assert out.shape == q.shape and lse.shape == (H, total)
        r0 = 0
        for L in lens:
            if L == 0:
                continue
            sl = slice(r0, r0 + L)
            qf, kf, vf = (t[sl].transpose(0, 1)[None].float().clone().requires_grad_() for t in (q, k, v))
            ref, _, _ = SO.streaming_attention_oracle(qf, kf, vf, c, back, None)
            ref.backward(do[sl].transpose(0, 1)[None].float())
            assert (out[sl].detach().cpu().float().transpose(0, 1)[None] - ref.detach()).abs().max() <= tol_o
            for gpu_grad, ref_grad in ((qs.grad, qf.grad), (ks.grad, kf.grad), (vs.grad, vf.grad)):
                assert (gpu_grad[sl].cpu().float().transpose(0, 1)[None] - ref_grad).abs().max() <= tol_g
            r0 += L


def test_packed_rejects_bad_offsets():
    from kernels_b200.streaming_attention import streaming_attention_varlen

    q = torch.randn(64, 2, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(AssertionError):
        streaming_attention_varlen(q, q, q, _cu([60]), 16, 1)  # cu_seqlens must end at `total`
