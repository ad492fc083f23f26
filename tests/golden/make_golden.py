"""Generate the golden fixtures in this folder from the UNMODIFIED reference project.

Run once in a CPU-only container that has the reference checked out::

    python tests/golden/make_golden.py /path/to/alexdremov-kernels

What runs is the reference's own code, imported from ``<ref>/src``:

* its torch oracle ``streaming_attention_reference`` / ``self_attention_reference`` —
  the hard-coded ``device="cuda"`` / ``.cuda()`` moves are redirected to the CPU by a
  ``TorchFunctionMode`` (arithmetic untouched);
* its Triton kernels through the op bodies (``attention_forward_adapter`` etc.) under
  ``TRITON_INTERPRET=1``.  The two autotuned launchers (``_streaming_attn_bwd_precompute``
  and ``softmax_kernel``) need a GPU driver to benchmark, so they are pinned to one launch
  configuration of their own search space; that changes tiling only, not arithmetic.

The fixtures are small ``.npz`` files holding inputs and the reference's outputs; the
tests in ``tests/test_oracle.py`` pin the CPU oracle to them and the GPU tests check the
CUDA path against them.
"""

from __future__ import annotations

import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402
from torch.overrides import TorchFunctionMode  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


class _CudaToCpu(TorchFunctionMode):
    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = dict(kwargs or {})
        dev = kwargs.get("device")
        if dev is not None and torch.device(dev).type == "cuda":
            kwargs["device"] = "cpu"
        return func(*args, **kwargs)


class _Pinned:
    """Stand-in for an autotuned launcher: always launches ``inner`` with fixed meta-parameters."""

    def __init__(self, inner, **meta):
        self.inner, self.meta = inner, meta

    def __getitem__(self, grid):
        return lambda *a, **k: self.inner[grid](*a, **self.meta, **k)


# (name, B, H, T, D, context, back, lens or None)
SA_CASES = [
    ("general", 2, 2, 80, 16, 10, 2, [80, 37]),
    ("perfect_tile", 1, 2, 96, 16, 32, 1, [70]),
    ("nolens_b0", 1, 1, 64, 32, 32, 0, None),
    ("odd_chunk_len_gt_T", 2, 1, 50, 64, 7, 3, [51, 5]),
    ("chunk_gt_T", 2, 1, 40, 16, 10000, 0, [40, 13]),
    ("chunk_1", 1, 2, 24, 16, 1, 5, None),
    ("back_huge", 1, 1, 70, 32, 16, 10000, [69]),
]

FA_CASES = [
    ("lens", 2, 2, 70, 16, [70, 33]),
    ("nolens", 1, 2, 48, 64, None),
    ("len_gt_T", 2, 1, 33, 128, [34, 1]),
]


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "src"))
    import streaming_attention.kernel as SA
    import self_attention.kernel as FA
    import softmax.kernel as SM

    torch.Tensor.cuda = lambda self, *a, **k: self
    SA._streaming_attn_bwd_precompute = _Pinned(SA._streaming_attn_bwd_precompute.fn, TILE_SIZE=32)
    SM.softmax_kernel = _Pinned(SM.softmax_kernel.fn, BLOCK_SIZE_ROWS=16, num_stages=2)

    out = {}
    for name, B, H, T, D, c, back, lens in SA_CASES:
        g = torch.Generator().manual_seed(1234 + len(out))
        q, k, v, do = (torch.randn(B, H, T, D, generator=g) for _ in range(4))
        lens_t = None if lens is None else torch.tensor(lens, dtype=torch.int32)
        scale = D ** -0.5
        with _CudaToCpu():
            qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
            ref, res_mask, sparsity = SA.streaming_attention_reference(qq, kk, vv, c, back, lens_t)
            do_m = do * res_mask.broadcast_to(do.shape)
            ref.backward(do_m)
        O, LSE = SA.attention_forward_adapter._init_fn(q, k, v, lens_t, c, back, scale, False, True, False, "ieee")
        dq, dk, dv = SA.attention_backward_adapter._init_fn(
            q, k, v, lens_t, O, LSE, do_m, c, back, scale, False, False, "ieee"
        )
        p = f"{name}/"
        out[p + "meta"] = np.array([B, H, T, D, c, back], dtype=np.int64)
        out[p + "lens"] = np.array([] if lens is None else lens, dtype=np.int32)
        for key, t in dict(q=q, k=k, v=v, do=do, ref_out=ref.detach(), ref_dq=qq.grad, ref_dk=kk.grad,
                           ref_dv=vv.grad, ker_out=O, ker_lse=LSE, ker_dq=dq, ker_dk=dk, ker_dv=dv).items():
            out[p + key] = t.numpy().astype(np.float32)
        out[p + "sparsity"] = np.array([sparsity], dtype=np.float64)
        err = (torch.nan_to_num(ref.detach()) * res_mask - O * res_mask).abs().max().item()
        print(f"streaming/{name}: kernel-vs-torch-reference fwd max err {err:.2e}")
    np.savez_compressed(os.path.join(HERE, "streaming_attention.npz"), **out)

    out = {}
    for name, B, H, T, D, lens in FA_CASES:
        g = torch.Generator().manual_seed(4321 + len(out))
        q, k, v = (torch.rand(B, H, T, D, generator=g) * 0.2 - 0.1 for _ in range(3))
        lens_t = None if lens is None else torch.tensor(lens, dtype=torch.int32)
        ref, _ = FA.self_attention_reference(q, k, v, lens_t)
        naive, _ = FA.self_attention_reference_naive(q, k, v, lens_t)
        ker = FA.attention_forward_adapter._init_fn(q, k, v, lens_t, D ** -0.5, False, False)
        p = f"{name}/"
        out[p + "meta"] = np.array([B, H, T, D], dtype=np.int64)
        out[p + "lens"] = np.array([] if lens is None else lens, dtype=np.int32)
        for key, t in dict(q=q, k=k, v=v, ref_out=ref, naive_out=naive, ker_out=ker).items():
            out[p + key] = t.numpy().astype(np.float32)
        print(f"self_attention/{name}: kernel-vs-reference max err {(torch.nan_to_num(ref) - ker).abs().max().item():.2e}")
    np.savez_compressed(os.path.join(HERE, "self_attention.npz"), **out)

    out = {}
    g = torch.Generator().manual_seed(99)
    for name, shape in [("ones_like_selfcheck", (13, 10, 19)), ("wide", (5, 300)), ("pow2", (8, 128))]:
        x = torch.ones(shape) if name.startswith("ones") else torch.randn(shape, generator=g) * 2.0
        out[f"{name}/x"] = x.numpy()
        out[f"{name}/naive"] = SM.softmax_naive(x).numpy()
        out[f"{name}/ker"] = SM.softmax(x).numpy()
        print(f"softmax/{name}: kernel-vs-naive max err {(SM.softmax(x) - SM.softmax_naive(x)).abs().max().item():.2e}")
    np.savez_compressed(os.path.join(HERE, "softmax.npz"), **out)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/alexdremov-kernels")
    main(sys.argv[1])
