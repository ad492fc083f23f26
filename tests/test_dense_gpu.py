"""GPU parity of the dense self-attention forward and the row softmax against the CPU oracle.

The self-attention grid mirrors ``tests/test_self_attention.py`` of the reference (dtype x lens
mode x layout x head_dim x batch x heads x time, inputs U[-0.1, 0.1], atol 1e-3 against the
oracle evaluated in the same low precision); the batch axis is trimmed where the O(T^2) CPU
oracle would take minutes.
"""

import itertools

import numpy as np
import pytest
import torch

from oracle import dense_oracle as DO

pytestmark = pytest.mark.gpu


def _self_attention_case(B, H, T, D, dtype, lens_mode, noncontiguous, rng):
    from kernels_b200.self_attention import self_attention

    mul = 2 if noncontiguous else 1
    shape = (B * mul, H * mul, T * mul, D * mul)
    q, k, v = ((torch.rand(shape) * 0.2 - 0.1).to(dtype) for _ in range(3))
    if noncontiguous:
        q, k, v = (t[1::2, 1::2, 1::2, 1::2] for t in (q, k, v))
    lens = None
    if lens_mode == "tricky":
        lens = torch.tensor(rng.choice([1, 2, 5, T + 1, T, max(T // 2, 1), max(T // 4, 1)], B), dtype=torch.int32)
    elif lens_mode == "random":
        lens = torch.from_numpy(rng.randint(1, T + 1, B).astype(np.int32))
    ref, res_mask = DO.self_attention_oracle(q.float(), k.float(), v.float(), lens)
    qg, kg, vg = (t.cuda() for t in (q, k, v))
    if noncontiguous:
        wide = [torch.zeros(shape, dtype=dtype, device="cuda") for _ in range(3)]
        for w, t in zip(wide, (qg, kg, vg)):
            w[1::2, 1::2, 1::2, 1::2] = t
        qg, kg, vg = (w[1::2, 1::2, 1::2, 1::2] for w in wide)
        assert qg.stride(-1) == 2
    out = self_attention(qg, kg, vg, lens.cuda() if lens is not None else None, autotune=False)
    assert out.is_contiguous() and out.dtype == dtype
    got = out.float().cpu()
    torch.testing.assert_close(got * res_mask, ref.to(dtype).float(), atol=1e-3, rtol=0)
    if lens is not None:
        assert (got * (~res_mask)).abs().max() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=str)
@pytest.mark.parametrize("D", [16, 128, 256])
@pytest.mark.parametrize("T", [1, 10, 16, 800, 1025])
def test_self_attention_reference_grid(dtype, D, T):
    rng = np.random.RandomState(T + D)
    torch.manual_seed(20)
    batches = [(1, 1), (40, 6), (64, 8)] if T <= 16 else [(1, 1), (3, 2)]
    for (B, H), lens_mode, nc in itertools.product(batches, ["none", "tricky", "random"], [False, True]):
        _self_attention_case(B, H, T, D, dtype, lens_mode, nc, rng)


@pytest.mark.parametrize("D", [32, 64])
def test_self_attention_other_head_dims_and_fp32(D):
    rng = np.random.RandomState(D)
    torch.manual_seed(1)
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        _self_attention_case(2, 3, 300, D, dtype, "random", False, rng)


def test_self_attention_golden(golden):
    from kernels_b200.self_attention import self_attention

    for name, c in golden("self_attention").items():
        lens = torch.tensor(c["lens"], dtype=torch.int32, device="cuda") if c["lens"].size else None
        q, k, v = (torch.from_numpy(c[x]).cuda() for x in "qkv")
        out = self_attention(q, k, v, lens).cpu()
        torch.testing.assert_close(out, torch.nan_to_num(torch.from_numpy(c["ref_out"])), atol=1e-6, rtol=0)
        torch.testing.assert_close(out, torch.from_numpy(c["ker_out"]), atol=1e-6, rtol=0)


@pytest.mark.parametrize("shape", [(13, 10, 19), (128, 256), (128, 2432), (7, 4096), (33, 4100), (5, 8192), (3, 20000),
                                   (1, 1), (0, 16), (4, 3, 257)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16], ids=str)
def test_softmax_matches_oracle(shape, dtype):
    from kernels_b200.softmax import softmax

    torch.manual_seed(0)
    x = (torch.randn(shape) * 2.0).to(dtype)
    y = softmax(x.cuda())
    assert y.shape == x.shape and y.dtype == dtype
    if x.numel() == 0:
        return
    ref = DO.softmax_oracle(x.float())
    tol = 1e-6 if dtype == torch.float32 else 4e-3
    torch.testing.assert_close(y.float().cpu(), ref, atol=tol, rtol=0)
    torch.testing.assert_close(y.float().sum(-1).cpu(), torch.ones(shape[:-1]), atol=2e-2, rtol=0)


def test_softmax_strided_rows_and_golden(golden):
    from kernels_b200.softmax import softmax

    base = torch.randn(64, 1024, device="cuda")
    view = base[:, :512]  # row stride 1024, 512 columns
    torch.testing.assert_close(softmax(view).cpu(), DO.softmax_oracle(view.cpu()), atol=1e-6, rtol=0)
    odd = base[:, 1:300]  # rows not 16-byte aligned: scalar kernel
    torch.testing.assert_close(softmax(odd).cpu(), DO.softmax_oracle(odd.cpu()), atol=1e-6, rtol=0)
    for name, c in golden("softmax").items():
        y = softmax(torch.from_numpy(c["x"]).cuda()).cpu()
        torch.testing.assert_close(y, torch.from_numpy(c["naive"]), atol=1e-6, rtol=0)
        torch.testing.assert_close(y, torch.from_numpy(c["ker"]), atol=1e-6, rtol=0)


def test_softmax_full_size_properties():
    """Benchmark shape [65536, 4096] fp32: rows sum to 1, order is preserved, shift-invariant."""
    from kernels_b200.softmax import softmax

    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(65536, 4096, device="cuda", generator=g) * 2.0
    y = softmax(x)
    assert torch.allclose(y.sum(-1), torch.ones(65536, device="cuda"), atol=1e-4)
    assert torch.equal(y.argmax(-1), x.argmax(-1))
    y2 = softmax(x + 3.0)
    assert torch.allclose(y, y2, atol=1e-6)
    rows = torch.tensor([0, 1, 31337, 65535])
    torch.testing.assert_close(y[rows.cuda()].cpu(), DO.softmax_oracle(x[rows.cuda()].cpu()), atol=1e-6, rtol=0)


def test_softmax_many_calls_side_stream_poisoned_output():
    """Regression guard for a result that could depend on timing or on what the output buffer held before:
    200 back-to-back calls of ``kb_softmax_fwd`` through the C ABI on a side stream, each with its own input
    and an output buffer filled with NaN beforehand, each compared element by element with the CPU oracle
    (the worst element's row / column is reported), and the first call's output compared bit for bit with a
    repeat of the same call at the end."""
    import ctypes

    from kernels_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    rows, cols, n_calls = 64, 4096, 200
    g = torch.Generator().manual_seed(7)
    xs_host = (torch.randn(n_calls, rows, cols, generator=g) * 2.0)
    xs = xs_host.to(dev)
    ys = torch.full((n_calls, rows, cols), float("nan"), device=dev)
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))

    def call(i, out):
        p = _lib.SoftmaxParams()
        p.x, p.y = xs[i].data_ptr(), out.data_ptr()
        p.rows, p.cols, p.x_row_stride, p.y_row_stride, p.dtype = rows, cols, cols, cols, _lib.KB_F32
        _lib.check(lib.kb_softmax_fwd(ctypes.byref(p), side.cuda_stream), "kb_softmax_fwd")

    for i in range(n_calls):
        call(i, ys[i])
    again = torch.full((rows, cols), float("nan"), device=dev)
    call(0, again)
    side.synchronize()
    got = ys.cpu()
    assert torch.equal(again.cpu(), got[0]), "the same call gave different bits"
    ref = DO.softmax_oracle(xs_host)
    err = (got - ref).abs()
    err[torch.isnan(got)] = float("inf")
    worst = int(err.argmax())
    i, r, c = worst // (rows * cols), (worst // cols) % rows, worst % cols
    assert float(err.max()) <= 1e-6, (
        f"softmax call {i} row {r} col {c}: got {float(got[i, r, c])!r}, oracle {float(ref[i, r, c])!r}, "
        f"|err| {float(err.max()):.3e}; {int((err > 1e-6).sum())} elements off, {int(torch.isnan(got).sum())} never written")
