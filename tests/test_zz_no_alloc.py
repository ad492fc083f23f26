"""GPU: the allocation-free backward entry point ``kb_sa_bwd_noalloc``.

Some hosts of this library may not allocate device memory around a call (a runtime plugin whose
execute hook only sees its bindings, a process whose arena owns the whole device, a loop that
cannot pay for cudaMalloc's device synchronisation).  For them the backward keeps its ``delta``
scratch in a fixed array inside the library.  This file checks, through the C ABI, that the
entry point gives the same gradients as ``kb_sa_bwd`` with caller-provided scratch, twice in a
row (the array is shared and keeps the previous call's contents), that it allocates nothing,
and that it refuses problems beyond the array's size.  It is collected last on purpose.
"""

import ctypes

import pytest
import torch

from kernels_b200 import _lib

pytestmark = pytest.mark.gpu


def _params(q, k, v, o, do, lse, dq, dk, dv, delta, lens, c, back):
    p = _lib.SaBwdParams()
    p.q, p.k, p.v, p.o, p.d_o = (_lib.tensor4(t) for t in (q, k, v, o, do))
    p.lse, p.dq, p.dk, p.dv = lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    p.delta_ws = delta.data_ptr() if delta is not None else None
    p.lens = lens.data_ptr() if lens is not None else None
    p.lens_stride = lens.stride(0) if lens is not None else 0
    p.B, p.H, p.T, p.D = q.shape
    p.dtype = _lib.dtype_code(q.dtype)
    p.context_size, p.back_contexts, p.sm_scale = c, back, float(q.shape[-1] ** -0.5)
    p.flags = 0
    p.status = _lib.status_words().data_ptr()
    return p


def _forward(q, k, v, lens, c, back):
    import kernels_b200.streaming_attention  # noqa: F401  (registers the operators)

    return torch.ops.alexdremov_streaming_attention.forward(
        q, k, v, lens, c, back, q.shape[-1] ** -0.5, False, True, False, "ieee")


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float16, 64), (torch.float32, 32)], ids=str)
def test_noalloc_backward_matches_regular_backward_twice(dtype, D):
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream(dev).cuda_stream
    B, H, T, c, back = 2, 3, 700, 48, 3
    for call in range(2):  # second round: other inputs, the shared array still holds the first round's delta
        g = torch.Generator(device="cpu").manual_seed(100 + call)
        q, k, v, do = (torch.randn(B, H, T, D, generator=g).to(dtype).to(dev) for _ in range(4))
        lens = torch.tensor([T, 333 + call], dtype=torch.int32, device=dev)
        o, lse = _forward(q, k, v, lens, c, back)

        ref = [torch.empty_like(q) for _ in range(3)]
        delta = torch.empty(B, H, T, dtype=torch.float32, device=dev)
        p_ref = _params(q, k, v, o, do, lse, *ref, delta, lens, c, back)
        _lib.check(lib.kb_sa_bwd(ctypes.byref(p_ref), stream), "kb_sa_bwd")

        got = [torch.full_like(q, float("nan")) for _ in range(3)]
        p_new = _params(q, k, v, o, do, lse, *got, None, lens, c, back)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        _lib.check(lib.kb_sa_bwd_noalloc(ctypes.byref(p_new), stream), "kb_sa_bwd_noalloc")
        torch.cuda.synchronize()
        if call == 1:  # the first call may load the kernels' code; after that nothing may be taken
            assert torch.cuda.mem_get_info(dev)[0] >= free_before
        _lib.check_device_status()
        # same kernels, same inputs, no atomics: the tolerance of the other tests holds trivially
        for name, a, b in zip(("dq", "dk", "dv"), got, ref):
            assert torch.isfinite(a).all(), name
            assert torch.equal(a, b), name


def test_noalloc_backward_rejects_problems_beyond_the_fixed_array():
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    t = torch.zeros(1, 1, 8, 64, dtype=torch.float16, device=dev)
    lse = torch.zeros(1, 1, 8, dtype=torch.float32, device=dev)
    p = _params(t, t, t, t, t, lse, t, t, t, None, None, 4, 1)
    p.B, p.H, p.T = 64, 32, 2048  # 4 Mi rows > KB_NOALLOC_MAX_ROWS; rejected before anything is read
    assert 64 * 32 * 2048 > _lib.KB_NOALLOC_MAX_ROWS
    rc = lib.kb_sa_bwd_noalloc(ctypes.byref(p), torch.cuda.current_stream(dev).cuda_stream)
    assert rc == 5
    with pytest.raises(RuntimeError, match="too large"):
        _lib.check(rc, "kb_sa_bwd_noalloc")
    assert lib.kb_sa_bwd_noalloc(None, None) == 1


def test_noalloc_backward_refuses_what_the_shared_array_cannot_serve():
    """Partial backwards (the per-kernel timing flags) would read an earlier call's delta out of the
    shared array; shared key/value heads and strided gradients are not served by its kernels."""
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream(dev).cuda_stream
    B, H, T, D = 1, 2, 256, 64
    q, k, v, do = (torch.randn(B, H, T, D, device=dev).half() for _ in range(4))
    o, lse = _forward(q, k, v, None, 32, 1)
    outs = [torch.full_like(q, float("nan")) for _ in range(3)]
    for flag in (_lib.KB_FLAG_BWD_SKIP_DQ, _lib.KB_FLAG_BWD_SKIP_DKDV, _lib.KB_FLAG_BWD_SKIP_DELTA):
        p = _params(q, k, v, o, do, lse, *outs, None, None, 32, 1)
        p.flags = flag
        assert lib.kb_sa_bwd_noalloc(ctypes.byref(p), stream) == 1
    p = _params(q, k, v, o, do, lse, *outs, None, None, 32, 1)
    p.H_kv = 1
    assert lib.kb_sa_bwd_noalloc(ctypes.byref(p), stream) == _lib.KB_ERR_UNSUPPORTED
    p = _params(q, k, v, o, do, lse, *outs, None, None, 32, 1)
    p.dq_stride[0], p.dq_stride[1], p.dq_stride[2] = H * T * D, T * D, D
    assert lib.kb_sa_bwd_noalloc(ctypes.byref(p), stream) == _lib.KB_ERR_UNSUPPORTED
    torch.cuda.synchronize()
    assert all(torch.isnan(t).all() for t in outs), "a refused call must not have launched anything"
