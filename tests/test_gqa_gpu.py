"""GPU: shared key/value heads (grouped-query attention), an extension of the reference's operator.

``k`` and ``v`` carry ``H_kv`` heads, ``H_kv`` dividing the ``H`` heads of ``q``; query head ``h`` reads
key/value head ``h // (H // H_kv)`` and ``dK`` / ``dV`` sum the contributions of a group's query heads.
The oracle is the CPU restatement of the reference applied to ``k`` / ``v`` with their heads repeated
(autograd then adds the group's gradients up).  16-bit inputs with head_dim 64 / 128 run natively on the
tcgen05 kernels (checked through the library's launch counter); everything else goes through the
operator's repeat-the-heads path.
"""

import pytest
import torch

from kernels_b200 import _lib
from oracle import streaming_attention_oracle as SO

pytestmark = pytest.mark.gpu


def _oracle(q, k, v, do, c, back, lens):
    group = q.shape[1] // k.shape[1]
    qf, kf, vf = (t.detach().float().clone().requires_grad_() for t in (q, k, v))
    out, res_mask, _ = SO.streaming_attention_oracle(
        qf, kf.repeat_interleave(group, dim=1), vf.repeat_interleave(group, dim=1), c, back, lens)
    out.backward(do.float() * res_mask.broadcast_to(do.shape))
    return torch.nan_to_num(out.detach()) * res_mask.broadcast_to(out.shape), qf.grad, kf.grad, vf.grad


@pytest.mark.parametrize("B,H,Hk,T,D,c,back,dtype,lens,native", [
    (2, 8, 2, 700, 128, 48, 3, torch.bfloat16, [700, 333], True),
    (1, 4, 1, 2048, 64, 256, 2, torch.float16, None, True),
    (2, 6, 3, 300, 128, 10, 5, torch.float16, [299, 17], True),
    (3, 4, 4, 260, 64, 128, 1, torch.float16, [260, 1, 130], True),   # H_kv = H: the plain operator
    (2, 4, 2, 200, 32, 24, 2, torch.float32, [200, 77], False),        # generic kernels: heads repeated
    (1, 6, 2, 130, 256, 64, 1, torch.float16, None, False),
])
def test_shared_kv_heads_match_oracle(B, H, Hk, T, D, c, back, dtype, lens, native):
    import kernels_b200.streaming_attention  # noqa: F401  (registers the operators)

    torch.manual_seed(5)
    q = torch.randn(B, H, T, D).to(dtype)
    k, v = (torch.randn(B, Hk, T, D).to(dtype) for _ in range(2))
    do = torch.randn(B, H, T, D).to(dtype)
    lens_t = None if lens is None else torch.tensor(lens, dtype=torch.int32)
    ref_out, ref_dq, ref_dk, ref_dv = _oracle(q, k, v, do, c, back, lens_t)
    res_mask = torch.ones(B, 1, T, 1, dtype=torch.bool)
    if lens_t is not None:
        res_mask = (torch.arange(T)[None] < lens_t[:, None])[:, None, :, None]

    qg, kg, vg = (t.cuda().requires_grad_() for t in (q, k, v))
    lens_g = None if lens_t is None else lens_t.cuda()
    n0 = _lib.launch_count()
    out, lse = torch.ops.alexdremov_streaming_attention.forward(qg, kg, vg, lens_g, c, back, D ** -0.5, False, True,
                                                                False, "ieee")
    n1 = _lib.launch_count()
    out.backward((do.float() * res_mask).to(dtype).cuda())
    torch.cuda.synchronize()
    n2 = _lib.launch_count()
    _lib.check_device_status()
    if native and Hk != H:
        assert (n1 - n0, n2 - n1) == (1, 3), "expected the tcgen05 forward and the delta / main / dQ kernels"
    assert kg.grad.shape == k.shape and vg.grad.shape == v.shape and out.shape == q.shape

    atol_f, atol_b = {torch.float32: (5e-6, 5e-5), torch.float16: (3e-3, 1e-2), torch.bfloat16: (2e-2, 6e-2)}[dtype]
    group = H // Hk
    got = out.detach().float().cpu()
    torch.testing.assert_close(got * res_mask, ref_out.to(dtype).float(), atol=atol_f, rtol=0)
    assert (got * (~res_mask)).abs().max() == 0
    for name, g, r, tol in (("dq", qg.grad, ref_dq, atol_b), ("dk", kg.grad, ref_dk, atol_b * group ** 0.5),
                            ("dv", vg.grad, ref_dv, atol_b * group ** 0.5)):
        gc = g.detach().float().cpu()
        assert torch.isfinite(gc).all(), name
        torch.testing.assert_close(gc, r.to(dtype).float(), atol=tol, rtol=0, msg=lambda m: f"{name}\n{m}")
        assert (gc * (~res_mask)).abs().max() == 0, name


def test_shared_kv_heads_through_public_api_and_twice_bitwise():
    from kernels_b200.streaming_attention import streaming_attention

    torch.manual_seed(9)
    q = torch.randn(2, 8, 1000, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k, v = (torch.randn(2, 2, 1000, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True) for _ in range(2))
    lens = torch.tensor([1000, 517], dtype=torch.int32, device="cuda")
    do = torch.randn_like(q)
    runs = []
    for _ in range(2):
        for t in (q, k, v):
            t.grad = None
        o = streaming_attention(q, k, v, lens, 256, 2)
        o.backward(do)
        runs.append([o.detach().clone(), q.grad.clone(), k.grad.clone(), v.grad.clone()])
    for a_, b_ in zip(*runs):
        assert torch.equal(a_, b_)
    # against the plain operator on repeated heads: same forward bits, gradients of a group add up
    k4, v4 = (t.detach().repeat_interleave(4, dim=1).requires_grad_() for t in (k, v))
    q4 = q.detach().clone().requires_grad_()
    o4 = streaming_attention(q4, k4, v4, lens, 256, 2)
    o4.backward(do)
    assert torch.equal(o4, runs[0][0]) and torch.equal(q4.grad, runs[0][1])
    for got, rep in ((runs[0][2], k4.grad), (runs[0][3], v4.grad)):
        want = rep.view(2, 2, 4, 1000, 128).float().sum(dim=2)
        torch.testing.assert_close(got.float(), want, atol=6e-2, rtol=2e-2)
