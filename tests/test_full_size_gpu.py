"""GPU parity at the benchmark's full sizes (the fp16 D=64 configuration, the long-sequence bf16
configuration and the per-sequence shape of the multi-GPU configuration).

The dense fp32 oracle cannot hold a T x T score matrix for every (batch, head) slice at these
sizes, so each configuration is checked two ways:

* a few (batch, head) slices against the banded fp64 oracle (an independent O(T * (back+1) * c)
  evaluation that ``tests/test_oracle.py`` pins to the dense restatement), with the benchmark
  contract's tolerances: output max-abs <= 2e-2, dQ / dK / dV relative L2 <= 2e-2;
* the WHOLE result through identities that hold for any size:
    - rows past ``lens`` are exact zeros in O, dQ, dK, dV;
    - with V = 1 every valid output row is 1 (the softmax weights of a row sum to 1);
    - sum_j dV[j, :] = sum_i dO[i, :] per (batch, head) (same reason, transposed);
    - sum(q * dQ) = sum(k * dK) per (batch, head): both equal scale * sum(dS * (Q K^T)).
"""

import pytest
import torch

from oracle import streaming_attention_oracle as SO

pytestmark = pytest.mark.gpu


def _api():
    from kernels_b200.streaming_attention import streaming_attention

    return streaming_attention


def _inputs(B, H, T, D, dtype, qk_scale, lens_range, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v, do = (torch.randn(B, H, T, D, device="cuda", generator=g, dtype=torch.float32) for _ in range(4))
    q, k = q * qk_scale, k * qk_scale
    lens = None
    if lens_range is not None:
        lens = torch.randint(lens_range[0], lens_range[1] + 1, (B,), generator=torch.Generator().manual_seed(seed),
                             dtype=torch.int32).cuda()
        valid = (torch.arange(T, device="cuda")[None] < lens[:, None])[:, None, :, None]
        do = do * valid  # the reference's tests mask dO the same way (tests/test_streaming_attention.py:155)
    return [t.to(dtype) for t in (q, k, v, do)], lens


def _run(q, k, v, do, lens, c, back):
    q, k, v = (t.detach().clone().requires_grad_() for t in (q, k, v))
    out, lse = _api()(q, k, v, lens, c, back, return_lse=True)
    out.backward(do)
    torch.cuda.synchronize()
    return out.detach(), lse.detach(), q.grad, k.grad, v.grad


def _check_slices(slices, q, k, v, do, lens, c, back, out, lse, dq, dk, dv):
    T = q.shape[2]
    for b, h in slices:
        L = T if lens is None else int(lens[b])
        ro, rl, rdq, rdk, rdv = SO.banded_fwd_bwd(q[b, h].float().cpu(), k[b, h].float().cpu(), v[b, h].float().cpu(),
                                                  do[b, h].float().cpu(), c, back, L)
        got_o = out[b, h].double().cpu()
        assert (got_o - ro).abs().max() <= 2e-2, ("out", b, h, float((got_o - ro).abs().max()))
        assert (lse[b, h, :L].double().cpu() - rl[:L]).abs().max() <= 2e-2, ("lse", b, h)
        for name, g_, r_ in (("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
            g64 = g_[b, h].double().cpu()
            rel = float((g64 - r_).norm() / r_.norm().clamp_min(1e-30))
            assert rel <= 2e-2, (name, b, h, rel)


def _check_identities(q, k, do, lens, out, dq, dk, dv, rel_tol):
    B, H, T, D = q.shape
    valid = torch.ones(B, 1, T, 1, dtype=torch.bool, device="cuda")
    if lens is not None:
        valid = (torch.arange(T, device="cuda")[None] < lens[:, None])[:, None, :, None]
    for name, t in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        assert torch.isfinite(t.float()).all(), name
        assert (t.float() * (~valid)).abs().max() == 0, f"{name}: rows past lens must be exact zeros"
    # column sums of dV against column sums of dO, per (batch, head)
    sv, sg = dv.double().sum(dim=2), (do.double() * valid).sum(dim=2)
    scale_ref = (do.double() * valid).abs().sum(dim=2).clamp_min(1e-30)
    assert ((sv - sg).abs() / scale_ref).max() <= rel_tol, float(((sv - sg).abs() / scale_ref).max())
    # sum(q * dq) = sum(k * dk), per (batch, head)
    a_ = (q.double() * dq.double()).sum(dim=(2, 3))
    b_ = (k.double() * dk.double()).sum(dim=(2, 3))
    denom = (q.double() * dq.double()).abs().sum(dim=(2, 3)).clamp_min(1e-30)
    assert ((a_ - b_).abs() / denom).max() <= rel_tol, float(((a_ - b_).abs() / denom).max())


def _check_rows_sum_to_one(q, k, lens, c, back, dtype):
    ones = torch.ones_like(q)
    out = _api()(q.detach(), k.detach(), ones, lens, c, back)
    torch.cuda.synchronize()
    B, H, T, D = q.shape
    valid = torch.ones(B, 1, T, 1, dtype=torch.bool, device="cuda")
    if lens is not None:
        valid = (torch.arange(T, device="cuda")[None] < lens[:, None])[:, None, :, None]
    tol = 2e-2 if dtype == torch.bfloat16 else 3e-3
    err = ((out.float() - 1.0) * valid).abs().max()
    assert err <= tol, float(err)
    assert (out.float() * (~valid)).abs().max() == 0


@pytest.mark.parametrize("name", ["config2", "config3", "config5_shape"])
def test_full_size(name):
    if name == "config2":   # fp16, 1 GPU: B=8 H=16 T=4096 D=64 c=128 back=4, q,k ~ N(0,1) * D^-0.25, lens ~ U[2048, 4096]
        B, H, T, D, c, back, dtype, qk, lr = 8, 16, 4096, 64, 128, 4, torch.float16, 64 ** -0.25, (2048, 4096)
        slices = [(0, 0), (3, 7), (7, 15)]
    elif name == "config3":  # bf16: B=4 H=32 T=16384 D=128 c=256 back=2, lens = T
        B, H, T, D, c, back, dtype, qk, lr = 4, 32, 16384, 128, 256, 2, torch.bfloat16, 1.0, None
        slices = [(0, 0), (2, 17), (3, 31)]
    else:                    # config 5's per-sequence shape (bf16 T=8192 D=128 c=64 back=8, lens ~ U[4096, 8192]), batch 4
        B, H, T, D, c, back, dtype, qk, lr = 4, 32, 8192, 128, 64, 8, torch.bfloat16, 1.0, (4096, 8192)
        slices = [(0, 0), (1, 9), (3, 31)]
    (q, k, v, do), lens = _inputs(B, H, T, D, dtype, qk, lr, seed=0)
    out, lse, dq, dk, dv = _run(q, k, v, do, lens, c, back)
    assert out.dtype == dtype and out.is_contiguous() and lse.shape == (B, H, T)
    _check_identities(q, k, do, lens, out, dq, dk, dv, rel_tol=2e-2 if dtype == torch.bfloat16 else 5e-3)
    _check_slices(slices, q, k, v, do, lens, c, back, out, lse, dq, dk, dv)
    del out, lse, dq, dk, dv
    _check_rows_sum_to_one(q, k, lens, c, back, dtype)
