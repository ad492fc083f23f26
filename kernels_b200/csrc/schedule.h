// Tile schedule of streaming attention: which KV tiles a q tile visits and which q tiles a
// KV tile receives gradient from.  One definition shared by the host planner (kb_sa_plan)
// and every kernel, so the schedule the tests check bit-exactly is the one the GPU walks.
//
// Mask: (i, j) is live iff  i < len, j < len and 0 <= i/c - j/c <= back
// (reference: src/streaming_attention/kernel.py:1540-1551).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define KB_HD __host__ __device__ __forceinline__
#else
#define KB_HD inline
#endif

struct KbTileRange {
  int32_t begin;
  int32_t end;  // one past the last tile; begin == end means nothing to visit
};

KB_HD int32_t kb_min_i32(int32_t a, int32_t b) { return a < b ? a : b; }
KB_HD int32_t kb_max_i32(int32_t a, int32_t b) { return a > b ? a : b; }
KB_HD int32_t kb_cdiv_i32(int32_t a, int32_t b) { return (a + b - 1) / b; }

// Clamp of the user's length to [0, T] (kernel.py:238-239) and of the chunk parameters to
// ranges in which all later products stay inside int32: a chunk longer than the sequence
// is one chunk, and looking back further than the number of chunks changes nothing.
KB_HD int32_t kb_clamp_len(int64_t len, int32_t T) { return len < 0 ? 0 : (len > T ? T : (int32_t)len); }
KB_HD int32_t kb_clamp_context(int64_t c, int32_t T) { return c > T ? kb_max_i32(T, 1) : (int32_t)c; }
KB_HD int32_t kb_clamp_back(int64_t back, int32_t T, int32_t c) {
  int32_t n = kb_cdiv_i32(kb_max_i32(T, 1), c);
  return back > n ? n : (int32_t)back;
}

// KV tiles visited by the q tile that starts at token q0 (kernel.py:243-244, 282-291).
KB_HD KbTileRange kb_fwd_kv_range(int32_t q0, int32_t tile_q, int32_t tile_k, int32_t len, int32_t c,
                                  int32_t back) {
  KbTileRange r = {0, 0};
  if (len <= q0) return r;
  int32_t min_ctx = q0 / c;
  r.begin = kb_max_i32(0, (min_ctx - back) * c) / tile_k;
  int32_t q_hi = kb_min_i32(q0 + tile_q, len);
  int32_t max_ctx = (q_hi - 1) / c;
  // (max_ctx + 1) * c can exceed int32 only if it exceeds len; compare in 64 bit.
  int64_t hi = (int64_t)(max_ctx + 1) * c;
  r.end = kb_cdiv_i32(hi < len ? (int32_t)hi : len, tile_k);
  return r;
}

// q tiles that send gradient to the KV tile starting at token k0 (kernel.py:1046-1054).
KB_HD KbTileRange kb_bwd_q_range(int32_t k0, int32_t tile_q, int32_t tile_k, int32_t len, int32_t c,
                                 int32_t back) {
  KbTileRange r = {0, 0};
  if (len <= k0) return r;
  int32_t min_ctx = k0 / c;
  r.begin = (min_ctx * c) / tile_q;
  int32_t k_max_tok = kb_min_i32(k0 + tile_k, len) - 1;
  int32_t max_ctx = k_max_tok / c;
  int64_t hi = (int64_t)(max_ctx + back + 1) * c;
  r.end = kb_cdiv_i32(hi < len ? (int32_t)hi : len, tile_q);
  return r;
}

// Division of a non-negative int32 by a positive int32 that is fixed for a launch, as one
// multiply-high, add and shift instead of the ~100-cycle integer-division sequence: the
// persistent kernels decode a work item (several divisions by the head count, the tile count
// and the chunk length) on their critical path every few tiles.  Exact for 0 <= n < 2^31.
struct KbFastDiv {
  uint32_t mul, shift, d;
};
inline KbFastDiv kb_fastdiv_make(int32_t divisor) {
  KbFastDiv f;
  f.d = (uint32_t)(divisor < 1 ? 1 : divisor);
  uint32_t s = 0;
  while (((uint64_t)1 << s) < f.d) ++s;  // s = ceil(log2 d)
  f.shift = s;
  f.mul = (uint32_t)((((uint64_t)1 << 32) * (((uint64_t)1 << s) - f.d)) / f.d + 1);
  return f;
}
KB_HD int32_t kb_fastdiv(int32_t n, const KbFastDiv& f) {
#if defined(__CUDA_ARCH__)
  const uint32_t hi = __umulhi((uint32_t)n, f.mul);
#else
  const uint32_t hi = (uint32_t)(((uint64_t)(uint32_t)n * f.mul) >> 32);
#endif
  return (int32_t)((hi + (uint32_t)n) >> f.shift);
}

// The two tile ranges above with the divisions by the chunk length done by kb_fastdiv (same
// results; the persistent kernels call these).
KB_HD KbTileRange kb_fwd_kv_range_fd(int32_t q0, int32_t tile_q, int32_t tile_k, int32_t len, int32_t c,
                                     int32_t back, const KbFastDiv& fc) {
  KbTileRange r = {0, 0};
  if (len <= q0) return r;
  int32_t min_ctx = kb_fastdiv(q0, fc);
  r.begin = kb_max_i32(0, (min_ctx - back) * c) / tile_k;
  int32_t q_hi = kb_min_i32(q0 + tile_q, len);
  int32_t max_ctx = kb_fastdiv(q_hi - 1, fc);
  int64_t hi = (int64_t)(max_ctx + 1) * c;
  r.end = kb_cdiv_i32(hi < len ? (int32_t)hi : len, tile_k);
  return r;
}
KB_HD KbTileRange kb_bwd_q_range_fd(int32_t k0, int32_t tile_q, int32_t tile_k, int32_t len, int32_t c,
                                    int32_t back, const KbFastDiv& fc) {
  KbTileRange r = {0, 0};
  if (len <= k0) return r;
  int32_t min_ctx = kb_fastdiv(k0, fc);
  r.begin = (min_ctx * c) / tile_q;
  int32_t k_max_tok = kb_min_i32(k0 + tile_k, len) - 1;
  int32_t max_ctx = kb_fastdiv(k_max_tok, fc);
  int64_t hi = (int64_t)(max_ctx + back + 1) * c;
  r.end = kb_cdiv_i32(hi < len ? (int32_t)hi : len, tile_q);
  return r;
}

// Element mask.  qc / kc are the chunk indices i/c and j/c.
KB_HD bool kb_live(int32_t i, int32_t j, int32_t qc, int32_t kc, int32_t len, int32_t back) {
  int32_t diff = qc - kc;
  return i < len && j < len && diff >= 0 && diff <= back;
}
