"""CPU oracle for streaming (chunked block-sparse) attention.  TEST INFRASTRUCTURE.

This module restates, for the host CPU, the torch masked-attention reference of
``alexdremov/kernels`` and the integer tile-range arithmetic of its kernels.  It
is the checker for the CUDA path: the product package never imports it.

Parity pin: ``tests/golden/`` holds outputs of the unmodified reference
(``src/streaming_attention/kernel.py``) produced in a CPU-only container by
``tests/golden/make_golden.py``; ``tests/test_oracle.py`` checks every function
here against those fixtures.

Reference lines followed (paths inside the reference project):

* mask + dense SDPA ............ ``src/streaming_attention/kernel.py:1533-1563``
* length clamp ``min(len, T)`` .. ``src/streaming_attention/kernel.py:238-239``
* forward KV tile range ........ ``src/streaming_attention/kernel.py:282-291`` and ``243-244``
* backward Q tile range ........ ``src/streaming_attention/kernel.py:1046-1054``
* base-2 LSE convention ........ ``src/streaming_attention/kernel.py:309, 407-408``
* test conventions (dO masking)  ``tests/test_streaming_attention.py:152-155, 183``
"""

from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

LOG2E = math.log2(math.e)


# --------------------------------------------------------------------------- #
# integer side: lengths, mask, tile ranges, useful-pair counts (bit-exact)
# --------------------------------------------------------------------------- #
def effective_lens(lens, B: int, T: int) -> np.ndarray:
    """``len_b = clamp(lens[b], 0, T)``, or ``T`` when ``lens`` is None.

    Follows ``src/streaming_attention/kernel.py:238-239`` (``min(seq_len, T)``); a
    non-positive length masks the whole sequence (every q tile takes the early
    exit of lines 243-244).
    """
    if lens is None:
        return np.full((B,), T, dtype=np.int64)
    arr = np.asarray(lens.detach().cpu().numpy() if isinstance(lens, torch.Tensor) else lens)
    return np.clip(arr.astype(np.int64), 0, T)


def chunk_mask(T: int, context_size: int, back_contexts: int) -> torch.Tensor:
    """``[T, T]`` bool: ``0 <= i//c - j//c <= back``  (kernel.py:1540-1542)."""
    blk = torch.div(torch.arange(T), context_size, rounding_mode="floor")
    diff = blk.unsqueeze(1) - blk.unsqueeze(0)
    return (diff >= 0) & (diff < back_contexts + 1)


def streaming_mask(T: int, context_size: int, back_contexts: int, lens_eff=None) -> torch.Tensor:
    """Full ``[B, 1, T, T]`` (or ``[T, T]`` without lens) attention mask (kernel.py:1540-1551)."""
    m = chunk_mask(T, context_size, back_contexts)
    if lens_eff is None:
        return m
    lens_t = torch.as_tensor(np.asarray(lens_eff), dtype=torch.int64)
    valid = torch.arange(T).unsqueeze(0) < lens_t.unsqueeze(-1)  # [B, T]
    pad = valid.unsqueeze(-1) & valid.unsqueeze(-2)  # [B, T, T]
    return m.unsqueeze(0).unsqueeze(0) & pad.unsqueeze(1)


def fwd_kv_tile_range(q0: int, tile_q: int, tile_k: int, seq_len: int, c: int, back: int):
    """KV tiles ``[start, end)`` a q tile starting at ``q0`` visits, or None when ``seq_len <= q0``.

    Integer restatement of ``src/streaming_attention/kernel.py:243-244, 282-291``.
    """
    if seq_len <= q0:
        return None
    q_min_ctx = q0 // c
    start = max(0, (q_min_ctx - back) * c) // tile_k
    q_hi = min(q0 + tile_q, seq_len)
    q_max_ctx = (q_hi - 1) // c
    end = -(-min((q_max_ctx + 1) * c, seq_len) // tile_k)
    return start, end


def bwd_q_tile_range(k0: int, tile_q: int, tile_k: int, seq_len: int, c: int, back: int):
    """Q tiles ``[start, end)`` a KV tile starting at ``k0`` receives gradient from.

    Integer restatement of ``src/streaming_attention/kernel.py:1046-1054``; returns
    None when the KV tile lies entirely in the padding.
    """
    if seq_len <= k0:
        return None
    k_min_ctx = k0 // c
    start = (k_min_ctx * c) // tile_q
    k_max_tok = min(k0 + tile_k, seq_len) - 1
    k_max_ctx = k_max_tok // c
    end = -(-min((k_max_ctx + back + 1) * c, seq_len) // tile_q)
    return start, end


def live_tiles_bruteforce(T: int, tile_q: int, tile_k: int, seq_len: int, c: int, back: int) -> np.ndarray:
    """``[nq, nk]`` bool: tile pair holds >= 1 unmasked element, derived from the dense mask."""
    m = streaming_mask(T, c, back, [seq_len])[0, 0].numpy()
    nq, nk = -(-T // tile_q), -(-T // tile_k)
    out = np.zeros((nq, nk), dtype=bool)
    for i in range(nq):
        for j in range(nk):
            out[i, j] = m[i * tile_q:(i + 1) * tile_q, j * tile_k:(j + 1) * tile_k].any()
    return out


def useful_pairs(seq_len: int, c: int, back: int) -> int:
    """Exact number of unmasked (i, j) pairs for one sequence of ``seq_len`` tokens."""
    if seq_len <= 0:
        return 0
    n_full, rem = divmod(seq_len, c)
    sizes = [c] * n_full + ([rem] if rem else [])
    pref = np.concatenate([[0], np.cumsum(sizes)])
    total = 0
    for ci, sz in enumerate(sizes):
        lo = max(0, ci - back)
        total += sz * int(pref[ci + 1] - pref[lo])
    return int(total)


# --------------------------------------------------------------------------- #
# floating-point side
# --------------------------------------------------------------------------- #
def streaming_attention_oracle(q, k, v, context_size, back_contexts, lens, scale=None):
    """Dense SDPA under the streaming mask on the tensors' own (CPU) device.

    Same signature and return triple ``(out, res_mask, sparsity_fraction)`` as the
    reference's ``streaming_attention_reference`` (kernel.py:1533-1563) with its three
    hard-coded ``.cuda()`` moves dropped.  Fully masked rows come out as 0.
    """
    T = q.shape[-2]
    attn_mask = chunk_mask(T, context_size, back_contexts).to(q.device)
    if lens is not None:
        key_padding = (torch.arange(T, device=q.device).unsqueeze(0) < lens.unsqueeze(-1)).unsqueeze(-1)
        both = key_padding & key_padding.transpose(-1, -2)
        attn_mask = attn_mask.unsqueeze(0).unsqueeze(0) & both.unsqueeze(1)
        res_mask = key_padding.unsqueeze(1)
    else:
        res_mask = torch.tensor([True], device=q.device)
    sparsity = attn_mask.sum().item() / attn_mask.numel()
    out = F.scaled_dot_product_attention(query=q, key=k, value=v, attn_mask=attn_mask, scale=scale)
    return out, res_mask, sparsity


def oracle_fwd_bwd(q, k, v, do, context_size, back_contexts, lens, scale=None):
    """Forward + autograd backward through :func:`streaming_attention_oracle`.

    ``do`` is multiplied by ``res_mask`` first, as ``tests/test_streaming_attention.py:155``
    does.  Returns ``(out, dq, dk, dv)`` as fp32 tensors; ``out`` is zeroed on padded rows.
    """
    qf, kf, vf = (t.detach().float().clone().requires_grad_() for t in (q, k, v))
    out, res_mask, _ = streaming_attention_oracle(qf, kf, vf, context_size, back_contexts, lens, scale)
    dof = do.detach().float() * res_mask.broadcast_to(do.shape)
    out.backward(dof)
    out = torch.nan_to_num(out.detach()) * res_mask.broadcast_to(out.shape)
    return out, qf.grad, kf.grad, vf.grad


def lse_base2_dense(q, k, context_size, back_contexts, lens, scale=None):
    """Base-2 log-sum-exp ``log2 sum_j 2^(s_ij * scale * log2 e)`` over unmasked j.

    Convention of ``src/streaming_attention/kernel.py:309, 407-408``.  Rows with no
    unmasked key hold ``-inf`` here; the kernels leave them unspecified, so compare
    only rows ``i < len``.
    """
    B, H, T, D = q.shape
    scale = D ** -0.5 if scale is None else scale
    lens_eff = effective_lens(lens, B, T) if lens is not None else None
    mask = streaming_mask(T, context_size, back_contexts, lens_eff)
    s = torch.einsum("bhid,bhjd->bhij", q.double(), k.double()) * (scale * LOG2E)
    s = s.masked_fill(~mask.broadcast_to(s.shape), float("-inf"))
    return (torch.logsumexp(s * math.log(2.0), dim=-1) / math.log(2.0)).float()


def banded_fwd_bwd(q, k, v, do, context_size, back_contexts, seq_len, scale=None, dtype=torch.float64):
    """Independent O(T * (back+1) * c) evaluation of ONE ``[T, D]`` slice, chunk by chunk.

    Never builds a ``T x T`` tensor, so it stands in for the dense oracle at the long
    sequence lengths of the benchmark; ``tests/test_oracle.py`` checks it against the
    dense restatement at small ``T``.  Returns ``(out, lse2, dq, dk, dv)`` in ``dtype``;
    rows/keys ``>= seq_len`` are zero (``lse2`` is 0 there).
    """
    T, D = q.shape
    scale = D ** -0.5 if scale is None else scale
    c, back = int(context_size), int(back_contexts)
    L = int(max(0, min(seq_len, T)))
    q_, k_, v_, do_ = (t.detach().to(dtype) for t in (q, k, v, do))
    out = torch.zeros(T, D, dtype=dtype)
    lse2 = torch.zeros(T, dtype=dtype)
    dq = torch.zeros(T, D, dtype=dtype)
    dk = torch.zeros(T, D, dtype=dtype)
    dv = torch.zeros(T, D, dtype=dtype)
    n_chunks = -(-L // c) if L > 0 else 0
    for ci in range(n_chunks):
        r0, r1 = ci * c, min((ci + 1) * c, L)
        k0, k1 = max(0, ci - back) * c, r1
        s = (q_[r0:r1] @ k_[k0:k1].T) * scale
        m = s.max(dim=-1, keepdim=True).values
        e = torch.exp(s - m)
        z = e.sum(dim=-1, keepdim=True)
        p = e / z
        o = p @ v_[k0:k1]
        out[r0:r1] = o
        lse2[r0:r1] = ((m + torch.log(z)) * LOG2E).squeeze(-1)
        g = do_[r0:r1]
        dv[k0:k1] += p.T @ g
        dp = g @ v_[k0:k1].T
        delta = (g * o).sum(dim=-1, keepdim=True)
        ds = p * (dp - delta) * scale
        dq[r0:r1] = ds @ k_[k0:k1]
        dk[k0:k1] += ds.T @ q_[r0:r1]
    return out, lse2, dq, dk, dv


# --------------------------------------------------------------------------- #
# deterministic synthetic inputs: the recipe lives with the product's benchmark helpers
# --------------------------------------------------------------------------- #
from kernels_b200.synthetic import make_lens, make_slice  # noqa: E402,F401
