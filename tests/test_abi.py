"""CPU: the C-ABI library loads, exports what include/kernels_b200.h declares, validates its
arguments, and its host planner reproduces the oracle's tile schedule bit for bit."""

import ctypes
import os
import re

import pytest
import torch

from kernels_b200 import _lib
from oracle import streaming_attention_oracle as SO

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "kernels_b200.h")).read()
    return re.findall(r"KB_API\s+[\w\s\*]+?\b(kb_\w+)\s*\(", text)


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared_symbols()
    assert len(names) >= 10 and set(names) == set(_lib.EXPORTS)
    for n in names:
        assert getattr(lib, n) is not None
    assert b"sm_100a" in lib.kb_version()


@pytest.mark.parametrize("T", [1, 10, 16, 800])
@pytest.mark.parametrize("c", [1, 10, 32, 256, 10000])
@pytest.mark.parametrize("back", [0, 2, 5, 10000])
@pytest.mark.parametrize("tiles", [(64, 64), (128, 128), (32, 32), (128, 64)])
def test_plan_is_bit_exact_against_oracle(T, c, back, tiles):
    tq, tk = tiles
    for L in sorted({1, 2, 5, c, c + 1, max(c - 1, 1), max(c * back, 1), T + 1, T, max(T // 2, 1), max(T // 4, 1)}):
        Le = min(L, T)
        fwd, bwd = _lib.plan(T, min(L, 2**31 - 1), c, back, tq, tk)
        for i, got in enumerate(fwd):
            want = SO.fwd_kv_tile_range(i * tq, tq, tk, Le, c, back)
            assert got == (want if want is not None else (0, 0)), (T, c, back, L, i)
        for j, got in enumerate(bwd):
            want = SO.bwd_q_tile_range(j * tk, tq, tk, Le, c, back)
            assert got == (want if want is not None else (0, 0)), (T, c, back, L, j)


def test_plan_handles_extreme_parameters_without_overflow():
    big = 2**31 - 1
    fwd, bwd = _lib.plan(1000, big, big, big, 128, 128)
    assert fwd == [(0, 8)] * 8 and bwd == [(0, 8)] * 8
    fwd, _ = _lib.plan(1000, 1000, 1, big, 128, 128)
    assert fwd == [(0, i + 1) for i in range(8)]
    fwd, _ = _lib.plan(1000, -5, 16, 2, 128, 128)
    assert fwd == [(0, 0)] * 8


def test_argument_validation_without_a_gpu():
    lib = _lib.load()
    assert lib.kb_sa_fwd(None, None) == 1
    p = _lib.SaFwdParams()
    p.B, p.H, p.T, p.D, p.dtype, p.context_size, p.back_contexts = 1, 1, 8, 48, _lib.KB_F16, 4, 1
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 2  # head_dim 48
    p.D, p.context_size = 64, 0
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 1  # context_size < 1
    p.context_size, p.back_contexts = 4, -1
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 1
    p.back_contexts, p.dtype = 1, 7
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 2  # dtype
    p.dtype = _lib.KB_F16
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 1  # null tensors
    p.T = 0
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 0  # empty problem: nothing to do
    b = _lib.SaBwdParams()
    b.B, b.H, b.T, b.D, b.dtype, b.context_size = 1, 1, 8, 64, _lib.KB_BF16, 4
    assert lib.kb_sa_bwd(ctypes.byref(b), None) == 1
    s = _lib.SoftmaxParams()
    s.rows, s.cols, s.dtype = 4, 4, _lib.KB_F32
    assert lib.kb_softmax_fwd(ctypes.byref(s), None) == 1
    s.rows = 0
    assert lib.kb_softmax_fwd(ctypes.byref(s), None) == 0
    assert b"bad argument" in lib.kb_strerror(1)
    with pytest.raises(RuntimeError, match="unsupported"):
        _lib.check(2, "x")


def _tile_constants():
    """The constants the kernels are compiled with (csrc/tiles.h), read from the source."""
    import re

    text = open(os.path.join(ROOT, "kernels_b200", "csrc", "tiles.h")).read()
    return {m.group(1): int(m.group(2)) for m in re.finditer(r"\b(k[A-Za-z]+)\s*=\s*(\d+)", text)}


def test_tile_table():
    """kb_sa_tile_config reports exactly the constants the kernels are compiled with."""
    k = _tile_constants()
    for dt in (torch.float16, torch.bfloat16):
        for D in (64, 128):
            for c in (64, 128, 256, 10000):
                want = {
                    0: (k["kFwdQRows"] * k["kFwdQTiles"], k["kFwdKeys"], k["kFwdStagesK"]),
                    1: (k["kTwoPassStationary"], k["kTwoPassStreamed"], k["kTwoPassStagesFirst"]),
                    2: (k["kTwoPassStreamed"], k["kTwoPassStationary"], k["kTwoPassStagesFirst"]),
                    3: (k["kMainQueries"], k["kMainKeys"], k["kMainStagesQ"]),
                    4: (k["kDqQueries"], k["kDqKeys"], k["kDqStages"]),
                }
                for which, (tq, tk, st) in want.items():
                    cfg = _lib.tile_config(dt, D, c, which=which)
                    assert cfg == dict(path=_lib.KB_PATH_SM100, tile_q=tq, tile_k=tk, stages=st), (dt, D, c, which, cfg)
    # the values this build commits (a change of the table shows up here as well as in tiles.h)
    assert _lib.tile_config(torch.bfloat16, 128, 256, which=0) == dict(path=1, tile_q=256, tile_k=128, stages=2)
    assert _lib.tile_config(torch.bfloat16, 128, 256, which=3) == dict(path=1, tile_q=128, tile_k=128, stages=2)
    assert _lib.tile_config(torch.bfloat16, 128, 256, which=4) == dict(path=1, tile_q=128, tile_k=128, stages=3)
    for D, tile in ((16, 64), (128, 64), (256, 32)):
        cfg = _lib.tile_config(torch.float32, D, 256)
        assert cfg == dict(path=_lib.KB_PATH_GENERIC, tile_q=tile, tile_k=tile, stages=1)
    cfg = _lib.tile_config(torch.float16, 64, 256, flags=_lib.KB_FLAG_FORCE_GENERIC)
    assert cfg["path"] == _lib.KB_PATH_GENERIC
    cfg = _lib.tile_config(torch.float16, 64, 256, unit_inner_stride=False)
    assert cfg["path"] == _lib.KB_PATH_GENERIC
    with pytest.raises(RuntimeError, match="bad argument"):
        _lib.tile_config(torch.float16, 64, 0)


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libkernels_b200.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()


def test_operators_have_no_cpu_path():
    from kernels_b200.softmax import softmax
    from kernels_b200.streaming_attention import streaming_attention  # noqa: F401

    q = torch.randn(1, 1, 8, 16)
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.alexdremov_streaming_attention.forward(q, q, q, None, 4, 1, 0.25, False, False, False, "ieee")
    with pytest.raises(RuntimeError):
        softmax(q)


def test_fake_implementations_trace_on_meta():
    """pt2 boundary: shapes/dtypes of the fake (meta) kernels, as the reference's fakes give them."""
    import kernels_b200.self_attention  # noqa: F401
    import kernels_b200.streaming_attention  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        q = torch.empty(3, 4, 50, 64, dtype=torch.float16, device="cuda").transpose(1, 2).transpose(1, 2)
        lens = torch.empty(3, dtype=torch.int32, device="cuda")
        o, lse = torch.ops.alexdremov_streaming_attention.forward(q, q, q, lens, 8, 2, 0.125, False, True, False, "ieee")
        assert o.shape == q.shape and o.dtype == q.dtype and o.is_contiguous()
        assert lse.shape == (3, 4, 50) and lse.dtype == torch.float32
        o2, lse2 = torch.ops.alexdremov_streaming_attention.forward(q, q, q, None, 8, 2, 0.125, False, False, False, "ieee")
        assert lse2.numel() == 0
        dq, dk, dv = torch.ops.alexdremov_streaming_attention.backward(
            q, q, q, lens, o, lse, o, 8, 2, 0.125, False, False, "ieee")
        assert dq.shape == dk.shape == dv.shape == q.shape
        o3 = torch.ops.alexdremov_flash_attention.forward(q, q, q, lens, 0.125, True, False)
        assert o3.shape == q.shape


def test_operator_schemas_keep_reference_argument_order():
    import kernels_b200.self_attention  # noqa: F401
    import kernels_b200.streaming_attention  # noqa: F401

    fwd = torch.ops.alexdremov_streaming_attention.forward.default._schema
    assert [a.name for a in fwd.arguments] == [
        "q", "k", "v", "lens", "context_size", "back_contexts", "sm_scale", "autotune", "return_lse",
        "prescale_qk", "precision"]
    bwd = torch.ops.alexdremov_streaming_attention.backward.default._schema
    assert [a.name for a in bwd.arguments] == [
        "q", "k", "v", "lens", "o", "lse", "do", "context_size", "back_contexts", "sm_scale", "autotune",
        "prescale_qk", "precision"]
    fa = torch.ops.alexdremov_flash_attention.forward.default._schema
    assert [a.name for a in fa.arguments] == ["q", "k", "v", "lens", "sm_scale", "autotune", "prescale"]


def test_forward_and_backward_schedules_name_the_same_tile_pairs():
    """The single-evaluation backward saves one dS tile per (key tile, query tile) pair of the
    TRANSPOSED schedule and its dQ kernel reads them by the FORWARD schedule, at slot
    ``query tile - first query tile of the key tile``: both schedules must list the same pairs."""
    import random

    rng = random.Random(7)
    for _ in range(1500):
        T = rng.choice([1, 5, 127, 128, 129, 300, 640, 777, 1000, 2048])
        c = rng.choice([1, 3, 10, 32, 48, 64, 100, 128, 129, 256, 300, 10000])
        back = rng.choice([0, 1, 2, 3, 5, 8, 10000])
        L = rng.choice([T, max(1, T // 2), rng.randint(0, T), T + 1])
        fwd, bwd = _lib.plan(T, L, c, back, 128, 128)
        pairs_f = {(i, j) for i, (b, e) in enumerate(fwd) for j in range(b, e)}
        pairs_b = {(i, j) for j, (b, e) in enumerate(bwd) for i in range(b, e)}
        assert pairs_f == pairs_b, (T, c, back, L)


def test_backward_workspace_size():
    lib = _lib.load()
    # bf16 B=4 H=32 T=16384 D=128 context 256 back 2: every 128-key tile meets at most 6 query tiles
    assert lib.kb_sa_bwd_workspace_bytes(4, 32, 16384, 128, _lib.KB_BF16, 256, 2) == 4 * 32 * 128 * 6 * 32768
    # the slot count is the widest row of the transposed schedule
    for T, c, back in [(700, 48, 3), (1000, 64, 8), (130, 128, 1), (2048, 10000, 0), (16, 10, 5)]:
        _, bwd = _lib.plan(T, T, c, back, 128, 128)
        w = max(e - b for b, e in bwd)
        assert lib.kb_sa_bwd_workspace_bytes(2, 3, T, 64, _lib.KB_F16, c, back) == 2 * 3 * len(bwd) * w * 32768
    # no single-evaluation kernel for fp32 or other head dims: no scratch wanted
    assert lib.kb_sa_bwd_workspace_bytes(2, 3, 700, 64, _lib.KB_F32, 48, 3) == 0
    assert lib.kb_sa_bwd_workspace_bytes(2, 3, 700, 32, _lib.KB_F16, 48, 3) == 0


def test_packed_batch_argument_validation_without_a_gpu():
    lib = _lib.load()
    assert lib.kb_sa_fwd_varlen(None, None) == 1 and lib.kb_sa_bwd_varlen(None, None) == 1
    p = _lib.SaVarlenParams()
    p.B, p.H, p.D, p.dtype, p.context_size, p.back_contexts = 0, 2, 64, _lib.KB_F16, 4, 1
    assert lib.kb_sa_fwd_varlen(ctypes.byref(p), None) == 0          # empty batch: nothing to do
    p.B = 2
    assert lib.kb_sa_fwd_varlen(ctypes.byref(p), None) == 1          # no cu_seqlens
    cu = (ctypes.c_int32 * 3)(0, 5, 3)
    p.cu_seqlens = ctypes.cast(cu, ctypes.c_void_p)
    assert lib.kb_sa_fwd_varlen(ctypes.byref(p), None) == 1          # decreasing
    cu[2] = 5
    cu[1] = 0
    cu2 = (ctypes.c_int32 * 3)(0, 0, 0)
    p.cu_seqlens = ctypes.cast(cu2, ctypes.c_void_p)
    assert lib.kb_sa_fwd_varlen(ctypes.byref(p), None) == 0          # only empty sequences
    p.cu_seqlens = ctypes.cast(cu, ctypes.c_void_p)
    assert lib.kb_sa_fwd_varlen(ctypes.byref(p), None) == 1          # null tensors
    p.H_kv = 3
    assert lib.kb_sa_fwd_varlen(ctypes.byref(p), None) == 1          # 3 key/value heads do not divide 2
    p.H_kv, p.D = 0, 32
    assert lib.kb_sa_fwd_varlen(ctypes.byref(p), None) == 2          # tcgen05 kernels only: head_dim 64 / 128
    p.D, p.dtype = 64, _lib.KB_F32
    assert lib.kb_sa_bwd_varlen(ctypes.byref(p), None) == 2
    p.dtype, p.context_size = _lib.KB_BF16, 0
    assert lib.kb_sa_bwd_varlen(ctypes.byref(p), None) == 1


def test_strided_outputs_are_validated_without_a_gpu():
    lib = _lib.load()
    buf = (ctypes.c_uint16 * 4096)()
    ptr = ctypes.cast(buf, ctypes.c_void_p)
    p = _lib.SaFwdParams()
    p.B, p.H, p.T, p.D, p.dtype, p.context_size, p.back_contexts = 1, 1, 8, 64, _lib.KB_F16, 4, 1
    for t in (p.q, p.k, p.v):
        t.data = ptr
        t.stride[0], t.stride[1], t.stride[2], t.stride[3] = 512, 512, 64, 1
    p.o = ptr
    p.sm_scale = 0.125
    p.o_stride[0], p.o_stride[1], p.o_stride[2] = 512, 64, 67
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 1                 # rows must stay 16-byte aligned
    p.o_stride[2] = 0
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 1                 # a strided output needs a row stride
    p.o_stride[2] = -64
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 1


def test_streaming_step_start_is_validated_without_a_gpu():
    lib = _lib.load()
    buf = (ctypes.c_uint16 * 4096)()
    ptr = ctypes.cast(buf, ctypes.c_void_p)
    p = _lib.SaFwdParams()
    p.B, p.H, p.T, p.D, p.dtype, p.context_size, p.back_contexts = 1, 1, 8, 64, _lib.KB_F16, 4, 1
    for t in (p.q, p.k, p.v):
        t.data = ptr
        t.stride[0], t.stride[1], t.stride[2], t.stride[3] = 512, 512, 64, 1
    p.o = ptr
    p.sm_scale = 0.125
    p.q_start = -1
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 1                 # before the first position
    p.q_start = 8
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 1                 # no query row left
    p.q_start, p.dtype = 4, _lib.KB_F32
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 2                 # tcgen05 kernels only


def test_packed_single_launch_arguments_are_validated_without_a_gpu():
    lib = _lib.load()
    buf = (ctypes.c_uint16 * 4096)()
    ptr = ctypes.cast(buf, ctypes.c_void_p)
    cu = (ctypes.c_int32 * 3)(0, 5, 8)
    p = _lib.SaFwdParams()
    p.B, p.H, p.T, p.D, p.dtype, p.context_size, p.back_contexts = 2, 1, 5, 64, _lib.KB_F16, 4, 1
    for t in (p.q, p.k, p.v):
        t.data = ptr
        t.stride[0], t.stride[1], t.stride[2], t.stride[3] = 0, 64, 64, 1
    p.o = ptr
    p.sm_scale = 0.125
    p.cu_seqlens = ctypes.cast(cu, ctypes.c_void_p)
    p.total_rows = 4
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 1                 # fewer rows than the longest sequence
    p.total_rows, p.q_start = 8, 1
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 1                 # a packed batch has no streaming step
    p.q_start = 0
    p.lens, p.lens_stride = ctypes.cast(cu, ctypes.c_void_p), 1
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 1                 # nor `lens`: the offsets give the lengths
    p.lens, p.dtype = None, _lib.KB_F32
    assert lib.kb_sa_fwd(ctypes.byref(p), None) == 2                 # tcgen05 kernels only
    assert lib.kb_fa_fwd(ctypes.byref(p), None) in (1, 2)            # the dense kernel takes no packed batch


def test_packed_backward_lane_count_is_validated_without_a_gpu():
    lib = _lib.load()
    buf = (ctypes.c_uint16 * 4096)()
    ptr = ctypes.cast(buf, ctypes.c_void_p).value
    cu = (ctypes.c_int32 * 3)(0, 5, 8)
    p = _lib.SaVarlenParams()
    p.B, p.H, p.D, p.dtype, p.context_size, p.back_contexts = 2, 1, 64, _lib.KB_F16, 4, 1
    p.cu_seqlens = ctypes.cast(cu, ctypes.c_void_p)
    for name in ("q", "k", "v", "o", "lse", "d_o", "dq", "dk", "dv", "delta_ws", "ds_ws"):
        setattr(p, name, ptr)
    p.ds_ws_bytes, p.sm_scale = 4096, 0.125
    p.lanes = 9
    assert lib.kb_sa_bwd_varlen(ctypes.byref(p), None) == 1          # at most eight lanes
