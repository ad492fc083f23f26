"""CPU: pin the oracle (oracle/) to the golden fixtures produced by the unmodified reference."""

import math

import numpy as np
import pytest
import torch

from oracle import dense_oracle as DO
from oracle import streaming_attention_oracle as SO


def _case_tensors(c):
    B, H, T, D, ctx, back = (int(x) for x in c["meta"])
    lens = torch.tensor(c["lens"], dtype=torch.int32) if c["lens"].size else None
    t = {k: torch.from_numpy(v) for k, v in c.items() if k not in ("meta", "lens", "sparsity")}
    return (B, H, T, D, ctx, back), lens, t


def test_streaming_oracle_matches_reference_outputs(golden):
    for name, c in golden("streaming_attention").items():
        (B, H, T, D, ctx, back), lens, t = _case_tensors(c)
        out, dq, dk, dv = SO.oracle_fwd_bwd(t["q"], t["k"], t["v"], t["do"], ctx, back, lens)
        res_mask = torch.ones(B, 1, T, 1, dtype=torch.bool)
        if lens is not None:
            res_mask = (torch.arange(T)[None] < lens[:, None])[:, None, :, None]
        # the reference's torch oracle (run unmodified on CPU): tight agreement
        ref_out = torch.nan_to_num(t["ref_out"]) * res_mask
        assert torch.allclose(out, ref_out, atol=2e-6, rtol=0), name
        for got, key in ((dq, "ref_dq"), (dk, "ref_dk"), (dv, "ref_dv")):
            assert torch.allclose(got, t[key], atol=1e-5, rtol=0), (name, key)
        # the reference's Triton kernels (interpreter): the tolerances of its own test-suite
        assert torch.allclose(out, t["ker_out"] * res_mask, atol=5e-6, rtol=0), name
        for got, key in ((dq, "ker_dq"), (dk, "ker_dk"), (dv, "ker_dv")):
            assert torch.allclose(got, t[key], atol=5e-5, rtol=0), (name, key)
        # sparsity fraction is integer arithmetic: exact
        _, _, sparsity = SO.streaming_attention_oracle(t["q"], t["k"], t["v"], ctx, back, lens)
        assert sparsity == float(c["sparsity"][0]), name


def test_lse_is_base2_and_matches_reference_kernel(golden):
    for name, c in golden("streaming_attention").items():
        (B, H, T, D, ctx, back), lens, t = _case_tensors(c)
        lse = SO.lse_base2_dense(t["q"], t["k"], ctx, back, lens)
        lens_eff = SO.effective_lens(lens, B, T)
        for b in range(B):
            L = int(lens_eff[b])
            assert torch.allclose(lse[b, :, :L], t["ker_lse"][b, :, :L], atol=2e-5, rtol=0), name


@pytest.mark.parametrize("T,c,back,L", [(80, 10, 2, 80), (80, 10, 2, 37), (96, 32, 1, 70), (50, 7, 3, 50),
                                        (40, 10000, 0, 13), (24, 1, 5, 24), (70, 16, 10000, 69), (33, 5, 0, 1)])
def test_banded_oracle_matches_dense(T, c, back, L):
    g = torch.Generator().manual_seed(T * 131 + c)
    D = 16
    q, k, v, do = (torch.randn(1, 1, T, D, generator=g, dtype=torch.float64) for _ in range(4))
    lens = torch.tensor([L], dtype=torch.int32)
    out, dq, dk, dv = SO.oracle_fwd_bwd(q.float(), k.float(), v.float(), do.float(), c, back, lens)
    o2, lse2, dq2, dk2, dv2 = SO.banded_fwd_bwd(q[0, 0], k[0, 0], v[0, 0], do[0, 0], c, back, L)
    assert torch.allclose(out[0, 0].double(), o2, atol=1e-5)
    assert torch.allclose(dq[0, 0].double(), dq2, atol=1e-4)
    assert torch.allclose(dk[0, 0].double(), dk2, atol=1e-4)
    assert torch.allclose(dv[0, 0].double(), dv2, atol=1e-4)
    lse_d = SO.lse_base2_dense(q.float(), k.float(), c, back, lens)[0, 0]
    assert torch.allclose(lse_d[:L].double(), lse2[:L], atol=1e-4)


@pytest.mark.parametrize("T", [1, 10, 16, 200])
@pytest.mark.parametrize("c", [1, 10, 32, 10000])
@pytest.mark.parametrize("back", [0, 5, 10000])
@pytest.mark.parametrize("tiles", [(32, 32), (64, 64), (128, 128), (64, 32), (16, 128)])
def test_tile_ranges_equal_bruteforce_live_set(T, c, back, tiles):
    """The contiguous ranges of the reference formulas are exactly the tiles with a live element."""
    tq, tk = tiles
    for L in sorted({1, 2, 5, c, c + 1, max(c - 1, 1), T, max(T // 2, 1), T + 1}):
        Le = min(L, T)
        live = SO.live_tiles_bruteforce(T, tq, tk, Le, min(c, max(T, 1)), back)
        nq, nk = live.shape
        for i in range(nq):
            r = SO.fwd_kv_tile_range(i * tq, tq, tk, Le, c, back)
            want = np.flatnonzero(live[i])
            if r is None:
                assert want.size == 0
            else:
                assert want.size and (r[0], r[1]) == (want[0], want[-1] + 1) and live[i, r[0]:r[1]].all()
        for j in range(nk):
            r = SO.bwd_q_tile_range(j * tk, tq, tk, Le, c, back)
            want = np.flatnonzero(live[:, j])
            if r is None:
                assert want.size == 0
            else:
                assert want.size and (r[0], r[1]) == (want[0], want[-1] + 1) and live[r[0]:r[1], j].all()


@pytest.mark.parametrize("T,c,back", [(64, 8, 2), (100, 7, 0), (33, 40, 3), (128, 16, 100)])
def test_useful_pairs_counts_mask(T, c, back):
    for L in (0, 1, min(c, T), T // 2, T):
        m = SO.streaming_mask(T, c, back, [L])
        assert SO.useful_pairs(L, c, back) == int(m.sum())
    n = T // c
    if T % c == 0 and n >= back + 1:
        assert SO.useful_pairs(T, c, back) == c * c * ((back + 1) * n - back * (back + 1) // 2)


def test_dense_oracles_match_reference(golden):
    for name, c in golden("self_attention").items():
        lens = torch.tensor(c["lens"], dtype=torch.int32) if c["lens"].size else None
        q, k, v = (torch.from_numpy(c[x]) for x in "qkv")
        out, _ = DO.self_attention_oracle(q, k, v, lens)
        naive, _ = DO.self_attention_oracle_naive(q, k, v, lens)
        for key in ("ref_out", "naive_out", "ker_out"):
            ref = torch.nan_to_num(torch.from_numpy(c[key]))
            assert torch.allclose(out, ref, atol=1e-6, rtol=0), (name, key)
            assert torch.allclose(naive, ref, atol=1e-6, rtol=0), (name, key)
    for name, c in golden("softmax").items():
        x = torch.from_numpy(c["x"])
        y = DO.softmax_oracle(x)
        assert torch.allclose(y, torch.from_numpy(c["naive"]), atol=1e-7, rtol=0)
        assert torch.allclose(y, torch.from_numpy(c["ker"]), atol=1e-6, rtol=0)
        assert torch.allclose(y, torch.softmax(x, -1), atol=1e-6, rtol=0)


def test_synthetic_inputs_are_shard_invariant():
    a = SO.make_slice(1, 3, 4, 8, 4, seed=0)
    b = SO.make_slice(1, 3, 4, 8, 4, seed=0)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    assert not torch.equal(a[0], SO.make_slice(1, 2, 4, 8, 4, seed=0)[0])
    lens = SO.make_lens(8, 256, 512, seed=0)
    assert lens.dtype == torch.int32 and int(lens.min()) >= 256 and int(lens.max()) <= 512
    assert math.isclose(SO.LOG2E, 1.4426950408889634)
