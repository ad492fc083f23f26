"""ctypes binding of ``lib/libkernels_b200.so`` (the C ABI declared in ``include/kernels_b200.h``).

There is no fallback: if the library has not been built, importing any operator of this
package raises, and every entry point raises ``RuntimeError`` on a non-zero status.
"""

from __future__ import annotations

import ctypes as C
import os

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "lib", "libkernels_b200.so")

KB_STATUS_WORDS = 4
KB_F32, KB_F16, KB_BF16 = 0, 1, 2
KB_FLAG_PRESCALE_QK, KB_FLAG_ALLOW_TF32, KB_FLAG_FORCE_GENERIC = 1, 2, 4
KB_FLAG_BWD_SKIP_DQ, KB_FLAG_BWD_SKIP_DKDV, KB_FLAG_BWD_TWO_PASS, KB_FLAG_BWD_SKIP_DELTA = 8, 16, 32, 64
KB_PATH_GENERIC, KB_PATH_SM100 = 0, 1
KB_ERR_UNSUPPORTED = 2
KB_NOALLOC_MAX_ROWS = 1 << 21

_DTYPES = {torch.float32: KB_F32, torch.float16: KB_F16, torch.bfloat16: KB_BF16}

EXPORTS = (
    "kb_sa_fwd", "kb_sa_fwd_fp8", "kb_sa_bwd", "kb_sa_bwd_workspace_bytes", "kb_sa_bwd_noalloc", "kb_sa_fwd_varlen", "kb_sa_bwd_varlen",
    "kb_sa_bwd_varlen_workspace_bytes", "kb_qkv_rope_proj", "kb_out_proj", "kb_fa_fwd", "kb_softmax_fwd", "kb_sa_plan", "kb_sa_tile_config",
    "kb_launch_count", "kb_strerror", "kb_last_cuda_error", "kb_version", "kb_selftest_wait_timeout",
)


class Tensor4(C.Structure):
    _fields_ = [("data", C.c_void_p), ("stride", C.c_int64 * 4)]


class SaFwdParams(C.Structure):
    _fields_ = [
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4),
        ("o", C.c_void_p), ("lse", C.c_void_p),
        ("lens", C.c_void_p), ("lens_stride", C.c_int64),
        ("B", C.c_int32), ("H", C.c_int32), ("T", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("context_size", C.c_int32), ("back_contexts", C.c_int32),
        ("sm_scale", C.c_float), ("flags", C.c_uint32), ("status", C.c_void_p),
        ("H_kv", C.c_int32),
        ("o_stride", C.c_int64 * 3), ("lse_stride", C.c_int64 * 2),
        ("q_start", C.c_int32),
        ("cu_seqlens", C.c_void_p), ("total_rows", C.c_int32),
    ]


class SaFwdFp8Params(C.Structure):
    _fields_ = [
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4),
        ("q_scale", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p), ("v_scale_max", C.c_void_p),
        ("o", C.c_void_p), ("lse", C.c_void_p), ("lens", C.c_void_p), ("lens_stride", C.c_int64),
        ("B", C.c_int32), ("H", C.c_int32), ("H_kv", C.c_int32), ("T", C.c_int32), ("D", C.c_int32),
        ("out_dtype", C.c_int32), ("context_size", C.c_int32), ("back_contexts", C.c_int32),
        ("sm_scale", C.c_float), ("flags", C.c_uint32), ("status", C.c_void_p),
    ]


class SaBwdParams(C.Structure):
    _fields_ = [
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("o", Tensor4), ("d_o", Tensor4),
        ("lse", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("delta_ws", C.c_void_p),
        ("lens", C.c_void_p), ("lens_stride", C.c_int64),
        ("B", C.c_int32), ("H", C.c_int32), ("T", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("context_size", C.c_int32), ("back_contexts", C.c_int32),
        ("sm_scale", C.c_float), ("flags", C.c_uint32), ("status", C.c_void_p),
        ("ds_ws", C.c_void_p), ("ds_ws_bytes", C.c_uint64),
        ("H_kv", C.c_int32),
        ("dq_stride", C.c_int64 * 3), ("dkv_stride", C.c_int64 * 3), ("lse_stride", C.c_int64 * 2),
        ("cu_seqlens", C.c_void_p), ("total_rows", C.c_int32),
    ]


class SaVarlenParams(C.Structure):
    """kb_sa_varlen_params: a packed batch, sequences one after the other along the token axis."""
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("lse", C.c_void_p),
        ("d_o", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("delta_ws", C.c_void_p), ("ds_ws", C.c_void_p), ("ds_ws_bytes", C.c_uint64),
        ("cu_seqlens", C.c_void_p),
        ("B", C.c_int32), ("H", C.c_int32), ("H_kv", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("context_size", C.c_int32), ("back_contexts", C.c_int32),
        ("sm_scale", C.c_float), ("flags", C.c_uint32), ("status", C.c_void_p),
        ("cu_seqlens_dev", C.c_void_p), ("lanes", C.c_uint32),
    ]


class QkvProjParams(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("w", C.c_void_p), ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p),
        ("B", C.c_int32), ("T", C.c_int32), ("E", C.c_int32), ("H", C.c_int32), ("H_kv", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("status", C.c_void_p),
    ]


class OutProjParams(C.Structure):
    _fields_ = [
        ("o", Tensor4), ("w", C.c_void_p), ("y", C.c_void_p),
        ("B", C.c_int32), ("T", C.c_int32), ("H", C.c_int32), ("D", C.c_int32), ("E_out", C.c_int32),
        ("dtype", C.c_int32), ("status", C.c_void_p),
    ]


class SoftmaxParams(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("y", C.c_void_p), ("rows", C.c_int64), ("cols", C.c_int64),
        ("x_row_stride", C.c_int64), ("y_row_stride", C.c_int64), ("dtype", C.c_int32),
    ]


_lib = None


def load() -> C.CDLL:
    """Load the shared library once; raise if it is missing (no CPU or eager fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m kernels_b200.build` "
            "(nvcc, sm_100a). kernels_b200 has no fallback path."
        )
    lib = C.CDLL(LIB_PATH)
    lib.kb_sa_fwd.argtypes = [C.POINTER(SaFwdParams), C.c_void_p]
    lib.kb_fa_fwd.argtypes = [C.POINTER(SaFwdParams), C.c_void_p]
    lib.kb_sa_bwd.argtypes = [C.POINTER(SaBwdParams), C.c_void_p]
    lib.kb_sa_fwd_fp8.argtypes = [C.POINTER(SaFwdFp8Params), C.c_void_p]
    lib.kb_sa_fwd_fp8.restype = C.c_int
    lib.kb_sa_bwd_noalloc.argtypes = [C.POINTER(SaBwdParams), C.c_void_p]
    lib.kb_sa_bwd_noalloc.restype = C.c_int
    lib.kb_sa_fwd_varlen.argtypes = [C.POINTER(SaVarlenParams), C.c_void_p]
    lib.kb_sa_bwd_varlen.argtypes = [C.POINTER(SaVarlenParams), C.c_void_p]
    lib.kb_sa_fwd_varlen.restype = lib.kb_sa_bwd_varlen.restype = C.c_int
    lib.kb_sa_bwd_workspace_bytes.argtypes = [C.c_int32] * 7
    lib.kb_sa_bwd_workspace_bytes.restype = C.c_uint64
    lib.kb_sa_bwd_varlen_workspace_bytes.argtypes = [C.c_int32] * 8
    lib.kb_sa_bwd_varlen_workspace_bytes.restype = C.c_uint64
    lib.kb_softmax_fwd.argtypes = [C.POINTER(SoftmaxParams), C.c_void_p]
    lib.kb_qkv_rope_proj.argtypes = [C.POINTER(QkvProjParams), C.c_void_p]
    lib.kb_out_proj.argtypes = [C.POINTER(OutProjParams), C.c_void_p]
    lib.kb_qkv_rope_proj.restype = lib.kb_out_proj.restype = C.c_int
    for f in (lib.kb_sa_fwd, lib.kb_fa_fwd, lib.kb_sa_bwd, lib.kb_softmax_fwd):
        f.restype = C.c_int
    lib.kb_sa_plan.argtypes = [C.c_int32] * 6 + [C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.kb_sa_plan.restype = C.c_int
    lib.kb_sa_tile_config.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_uint32, C.c_int32, C.c_int32] + [
        C.POINTER(C.c_int32)
    ] * 4
    lib.kb_sa_tile_config.restype = C.c_int
    lib.kb_launch_count.restype = C.c_int64
    lib.kb_selftest_wait_timeout.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
    lib.kb_selftest_wait_timeout.restype = C.c_int
    for f in (lib.kb_strerror, lib.kb_last_cuda_error, lib.kb_version):
        f.restype = C.c_char_p
    lib.kb_strerror.argtypes = [C.c_int]
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        lib = load()
        msg = lib.kb_strerror(rc).decode()
        detail = lib.kb_last_cuda_error().decode()
        raise RuntimeError(f"{what}: {msg}" + (f" [{detail}]" if detail and rc == 3 else ""))


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise RuntimeError(f"kernels_b200: unsupported dtype {dtype}") from None


def tensor4(t: torch.Tensor) -> Tensor4:
    out = Tensor4()
    out.data = t.data_ptr()
    for i in range(4):
        out.stride[i] = t.stride(i)
    return out


def launch_count() -> int:
    return int(load().kb_launch_count())


# Pinned status words the kernels can write when a bounded device-side wait gives up.
_status = None


def status_words() -> torch.Tensor:
    global _status
    if _status is None:
        _status = torch.zeros(KB_STATUS_WORDS, dtype=torch.int32).pin_memory()
    return _status


def check_device_status() -> None:
    """Raise if any kernel reported a timed-out wait.  Call after synchronising the stream."""
    if _status is not None and int(_status[0]) != 0:
        words = _status.tolist()
        _status.zero_()
        raise RuntimeError(f"kernels_b200: a device-side wait timed out (status words {words})")


def plan(T: int, seq_len: int, context_size: int, back_contexts: int, tile_q: int, tile_k: int):
    """Host tile schedule: ``(fwd_ranges[nq, 2], bwd_ranges[nk, 2])`` as nested lists."""
    lib = load()
    nq, nk = -(-T // tile_q), -(-T // tile_k)
    fwd = (C.c_int32 * (2 * max(nq, 1)))()
    bwd = (C.c_int32 * (2 * max(nk, 1)))()
    rc = lib.kb_sa_plan(T, seq_len, context_size, back_contexts, tile_q, tile_k, fwd, bwd)
    if rc < 0:
        check(-rc, "kb_sa_plan")
    return [(fwd[2 * i], fwd[2 * i + 1]) for i in range(nq)], [(bwd[2 * j], bwd[2 * j + 1]) for j in range(nk)]


def tile_config(dtype: torch.dtype, D: int, context_size: int, which: int = 0, flags: int = 0, unit_inner_stride=True):
    """Committed tile table: ``dict(path, tile_q, tile_k, stages)`` for forward (0), the two-pass backward's
    dQ pass (1) and dK/dV pass (2), the single-evaluation backward's main kernel (3) and dQ kernel (4)."""
    lib = load()
    vals = [C.c_int32() for _ in range(4)]
    rc = lib.kb_sa_tile_config(dtype_code(dtype), D, context_size, flags, int(unit_inner_stride), which,
                               *[C.byref(v) for v in vals])
    check(rc, "kb_sa_tile_config")
    return dict(path=vals[0].value, tile_q=vals[1].value, tile_k=vals[2].value, stages=vals[3].value)
