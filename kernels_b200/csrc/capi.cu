// extern "C" surface of the library (declared in include/kernels_b200.h): argument
// validation, kernel-family selection and the host-side schedule planner.
#include <atomic>
#include <mutex>
#include <cstdio>
#include <cstring>

#include "common.cuh"
#include "tiles.h"

namespace kb {

namespace {
std::atomic<int64_t> g_launches{0};
thread_local char g_cuda_error[256] = "";
}  // namespace

void set_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%s)", where, cudaGetErrorName(e), cudaGetErrorString(e));
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

namespace {

bool head_dim_ok(int32_t D) { return D == 16 || D == 32 || D == 64 || D == 128 || D == 256; }
bool dtype_ok(int32_t t) { return t == KB_F32 || t == KB_F16 || t == KB_BF16; }

template <typename P>
int check_common(const P* p) {
  if (!p) return KB_ERR_BAD_ARGUMENT;
  if (p->B < 0 || p->H < 0 || p->T < 0) return KB_ERR_BAD_ARGUMENT;
  if (!dtype_ok(p->dtype) || !head_dim_ok(p->D)) return KB_ERR_UNSUPPORTED;
  if (p->B > 65535 || p->H > 65535) return KB_ERR_TOO_LARGE;
  if ((int64_t)p->T > (int64_t)1 << 30) return KB_ERR_TOO_LARGE;
  return KB_OK;
}

bool empty(int32_t B, int32_t H, int32_t T) { return B == 0 || H == 0 || T == 0; }

// The tcgen05 path wants 16-bit inputs, a head dim of 64 or 128, unit stride along the head
// dim and 16-byte aligned rows (TMA's requirements on the tensor map).
bool tma_ok(const kb_tensor4& t, size_t elsize) {
  if (t.stride[3] != 1) return false;
  if (reinterpret_cast<uintptr_t>(t.data) % 16) return false;
  for (int i = 0; i < 3; ++i)
    if ((t.stride[i] * (int64_t)elsize) % 16 || t.stride[i] < 0) return false;
  return true;
}

#ifdef KB_HAVE_SM100
bool sm100_shape_ok(int32_t dtype, int32_t D, uint32_t flags) {
  return (dtype == KB_F16 || dtype == KB_BF16) && (D == 64 || D == 128) && !(flags & KB_FLAG_FORCE_GENERIC);
}
#endif

int select_fwd_path(const kb_sa_fwd_params& p) {
#ifdef KB_HAVE_SM100
  if (sm100_shape_ok(p.dtype, p.D, p.flags) && tma_ok(p.q, 2) && tma_ok(p.k, 2) && tma_ok(p.v, 2)) return KB_PATH_SM100;
#endif
  return KB_PATH_GENERIC;
}

int select_bwd_path(const kb_sa_bwd_params& p) {
#ifdef KB_HAVE_SM100_BWD
  if (sm100_shape_ok(p.dtype, p.D, p.flags) && tma_ok(p.q, 2) && tma_ok(p.k, 2) && tma_ok(p.v, 2) &&
      tma_ok(p.o, 2) && tma_ok(p.d_o, 2))
    return KB_PATH_SM100;
#endif
  return KB_PATH_GENERIC;
}

// heads of k / v: H unless the caller asked for shared key/value heads; -1 if the request is invalid
template <typename P>
int32_t kv_heads(const P* p) {
  if (p->H_kv == 0 || p->H_kv == p->H) return p->H;
  if (p->H_kv < 0 || p->H_kv > p->H || p->H % p->H_kv) return -1;
  return p->H_kv;
}

template <int N>
bool any_stride(const int64_t (&st)[N]) {
  for (int i = 0; i < N; ++i)
    if (st[i]) return true;
  return false;
}
// a strided output: 16-byte aligned rows (the tensor map's and the plain stores' requirement)
bool out_stride_ok(const int64_t (&st)[3]) {
  if (!any_stride(st)) return true;
  for (int i = 0; i < 3; ++i)
    if (st[i] < 0 || st[i] % 8) return false;
  return st[2] > 0;
}

int run_fwd(const kb_sa_fwd_params* p, void* stream, bool dense) {
  int rc = check_common(p);
  if (rc) return rc;
  if (kv_heads(p) < 0) return KB_ERR_BAD_ARGUMENT;
  if (!dense && (p->context_size < 1 || p->back_contexts < 0)) return KB_ERR_BAD_ARGUMENT;
  if (empty(p->B, p->H, p->T)) return KB_OK;
  if (!p->q.data || !p->k.data || !p->v.data || !p->o) return KB_ERR_BAD_ARGUMENT;
  if (!out_stride_ok(p->o_stride) || p->lse_stride[0] < 0 || p->lse_stride[1] < 0) return KB_ERR_BAD_ARGUMENT;
  if (p->q_start < 0 || p->q_start >= p->T) return KB_ERR_BAD_ARGUMENT;
  if (p->cu_seqlens && (dense || p->lens || p->q_start || p->total_rows < p->T)) return KB_ERR_BAD_ARGUMENT;
  const bool strided_out = any_stride(p->o_stride) || any_stride(p->lse_stride);
  const int32_t c = dense ? kb_max_i32(p->T, 1) : kb_clamp_context(p->context_size, p->T);
  const int32_t back = dense ? 0 : kb_clamp_back(p->back_contexts, p->T, c);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#ifdef KB_HAVE_SM100
  if (select_fwd_path(*p) == KB_PATH_SM100) {
    // KB_ERR_UNSUPPORTED from the tcgen05 launcher means "this layout has no tensor map":
    // nothing was launched, the generic kernels take over.
    const int rc = sa_fwd_sm100(*p, c, back, s);
    if (rc != KB_ERR_UNSUPPORTED) return rc;
  }
#endif
  // the generic kernels want one K/V head per query head, contiguous outputs and every query row
  if (kv_heads(p) != p->H || strided_out || p->q_start || p->cu_seqlens) return KB_ERR_UNSUPPORTED;
  return sa_fwd_generic(*p, c, back, s);
}

}  // namespace
}  // namespace kb

extern "C" {

int kb_sa_fwd(const kb_sa_fwd_params* p, void* stream) { return kb::run_fwd(p, stream, /*dense=*/false); }

int kb_fa_fwd(const kb_sa_fwd_params* p, void* stream) { return kb::run_fwd(p, stream, /*dense=*/true); }

int kb_sa_fwd_fp8(const kb_sa_fwd_fp8_params* p, void* stream) {
  if (!p || p->B < 0 || p->H < 1 || p->T < 0 || p->context_size < 1 || p->back_contexts < 0) return KB_ERR_BAD_ARGUMENT;
  const int32_t Hk = p->H_kv > 0 ? p->H_kv : p->H;
  if (Hk > p->H || p->H % Hk) return KB_ERR_BAD_ARGUMENT;
  if (p->D != 128 || (p->out_dtype != KB_F16 && p->out_dtype != KB_BF16)) return KB_ERR_UNSUPPORTED;
  if (p->B > 65535 || p->H > 65535 || (int64_t)p->T > (int64_t)1 << 30) return KB_ERR_TOO_LARGE;
  if (kb::empty(p->B, p->H, p->T)) return KB_OK;
  if (!p->q.data || !p->k.data || !p->v.data || !p->o || !p->q_scale || !p->k_scale || !p->v_scale || !p->v_scale_max)
    return KB_ERR_BAD_ARGUMENT;
#ifdef KB_HAVE_SM100
  const int32_t c = kb_clamp_context(p->context_size, p->T);
  const int32_t back = kb_clamp_back(p->back_contexts, p->T, c);
  kb_sa_fwd_fp8_params q = *p;
  q.H_kv = Hk;
  return kb::sa_fwd_sm100_fp8(q, c, back, static_cast<cudaStream_t>(stream));
#else
  (void)stream;
  return KB_ERR_UNSUPPORTED;
#endif
}

int kb_sa_bwd(const kb_sa_bwd_params* p, void* stream) {
  int rc = kb::check_common(p);
  if (rc) return rc;
  if (p->context_size < 1 || p->back_contexts < 0 || kb::kv_heads(p) < 0) return KB_ERR_BAD_ARGUMENT;
  if (kb::empty(p->B, p->H, p->T)) return KB_OK;
  if (!p->q.data || !p->k.data || !p->v.data || !p->o.data || !p->d_o.data || !p->lse || !p->dq || !p->dk ||
      !p->dv || !p->delta_ws)
    return KB_ERR_BAD_ARGUMENT;
  if (!kb::out_stride_ok(p->dq_stride) || !kb::out_stride_ok(p->dkv_stride) || p->lse_stride[0] < 0 || p->lse_stride[1] < 0)
    return KB_ERR_BAD_ARGUMENT;
  if (p->cu_seqlens && (p->lens || p->total_rows < p->T || !p->ds_ws)) return KB_ERR_BAD_ARGUMENT;
  const bool strided_out = kb::any_stride(p->dq_stride) || kb::any_stride(p->dkv_stride) || kb::any_stride(p->lse_stride);
  const int32_t c = kb_clamp_context(p->context_size, p->T);
  const int32_t back = kb_clamp_back(p->back_contexts, p->T, c);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#ifdef KB_HAVE_SM100_BWD
  if (kb::select_bwd_path(*p) == KB_PATH_SM100) {
#ifdef KB_HAVE_SM100_BWD_FUSED
    // scores evaluated once when the caller brought the dS scratch; "unsupported" = nothing launched
    if (p->ds_ws && !(p->flags & KB_FLAG_BWD_TWO_PASS)) {
      const int rc = kb::sa_bwd_fused_sm100(*p, c, back, s);
      if (rc != KB_ERR_UNSUPPORTED) return rc;
    }
#endif
    // shared K/V heads, strided gradients and packed batches: single-evaluation kernels only
    if (kb::kv_heads(p) != p->H || strided_out || p->cu_seqlens) return KB_ERR_UNSUPPORTED;
    const int rc = kb::sa_bwd_sm100(*p, c, back, s);
    if (rc != KB_ERR_UNSUPPORTED) return rc;
  }
#endif
  if (kb::kv_heads(p) != p->H || strided_out || p->cu_seqlens) return KB_ERR_UNSUPPORTED;
  return kb::sa_bwd_generic(*p, c, back, s);
}

// Packed batch: one call of the entry points above per sequence, over strided views of the packed tensors.
namespace {
int check_varlen(const kb_sa_varlen_params* p, bool backward) {
  if (!p || p->B < 0 || p->H < 1 || p->context_size < 1 || p->back_contexts < 0) return KB_ERR_BAD_ARGUMENT;
  const int32_t Hk = p->H_kv > 0 ? p->H_kv : p->H;
  if (Hk > p->H || p->H % Hk) return KB_ERR_BAD_ARGUMENT;
  if (!kb::sm100_shape_ok(p->dtype, p->D, p->flags)) return KB_ERR_UNSUPPORTED;
  if (p->B == 0) return KB_OK;
  if (!p->cu_seqlens || p->cu_seqlens[0] != 0) return KB_ERR_BAD_ARGUMENT;
  for (int32_t b = 0; b < p->B; ++b)
    if (p->cu_seqlens[b + 1] < p->cu_seqlens[b]) return KB_ERR_BAD_ARGUMENT;
  if (p->cu_seqlens[p->B] == 0) return KB_OK;
  if (!p->q || !p->k || !p->v || !p->o) return KB_ERR_BAD_ARGUMENT;
  if (backward && (!p->lse || !p->d_o || !p->dq || !p->dk || !p->dv || !p->delta_ws || !p->ds_ws)) return KB_ERR_BAD_ARGUMENT;
  return KB_OK;
}
// rows [row0, ...) of a packed [total, heads, D] tensor as a [1, heads, len, D] view
kb_tensor4 packed_view(const void* base, int64_t row0, int32_t heads, int32_t D) {
  kb_tensor4 t;
  t.data = static_cast<const uint16_t*>(base) + row0 * heads * D;
  t.stride[0] = 0;  // extent 1
  t.stride[1] = D;
  t.stride[2] = (int64_t)heads * D;
  t.stride[3] = 1;
  return t;
}
}  // namespace

int kb_sa_fwd_varlen(const kb_sa_varlen_params* p, void* stream) {
  int rc = check_varlen(p, false);
  if (rc || p->B == 0) return rc;
  const int32_t Hk = p->H_kv > 0 ? p->H_kv : p->H, D = p->D;
  const int64_t total = p->cu_seqlens[p->B];
  if (total == 0) return KB_OK;
  if (p->cu_seqlens_dev) {
    // one launch: the kernel finds every sequence's first row and length in the device copy of the offsets
    int32_t max_len = 0;
    for (int32_t b = 0; b < p->B; ++b) max_len = kb_max_i32(max_len, p->cu_seqlens[b + 1] - p->cu_seqlens[b]);
    kb_sa_fwd_params f = {};
    f.q = packed_view(p->q, 0, p->H, D);
    f.k = packed_view(p->k, 0, Hk, D);
    f.v = packed_view(p->v, 0, Hk, D);
    f.o = p->o;
    f.o_stride[0] = total * p->H * D, f.o_stride[1] = D, f.o_stride[2] = (int64_t)p->H * D;
    f.lse = p->lse;
    f.lse_stride[0] = total * p->H, f.lse_stride[1] = total;
    f.B = p->B, f.H = p->H, f.T = max_len, f.D = D, f.H_kv = Hk;
    f.dtype = p->dtype, f.context_size = p->context_size, f.back_contexts = p->back_contexts;
    f.sm_scale = p->sm_scale, f.flags = p->flags, f.status = p->status;
    f.cu_seqlens = p->cu_seqlens_dev, f.total_rows = (int32_t)total;
    return kb_sa_fwd(&f, stream);
  }
  for (int32_t b = 0; b < p->B; ++b) {
    const int64_t r0 = p->cu_seqlens[b];
    const int32_t len = p->cu_seqlens[b + 1] - p->cu_seqlens[b];
    if (len == 0) continue;
    kb_sa_fwd_params f = {};
    f.q = packed_view(p->q, r0, p->H, D);
    f.k = packed_view(p->k, r0, Hk, D);
    f.v = packed_view(p->v, r0, Hk, D);
    f.o = static_cast<uint16_t*>(p->o) + r0 * p->H * D;
    f.o_stride[0] = (int64_t)len * p->H * D, f.o_stride[1] = D, f.o_stride[2] = (int64_t)p->H * D;
    f.lse = p->lse ? p->lse + r0 : nullptr;
    f.lse_stride[0] = total * p->H, f.lse_stride[1] = total;
    f.B = 1, f.H = p->H, f.T = len, f.D = D, f.H_kv = Hk;
    f.dtype = p->dtype, f.context_size = p->context_size, f.back_contexts = p->back_contexts;
    f.sm_scale = p->sm_scale, f.flags = p->flags, f.status = p->status;
    rc = kb_sa_fwd(&f, stream);
    if (rc) return rc;
  }
  return KB_OK;
}

// Lanes of the packed backward: streams of the library's own on which the per-sequence launches of different
// sequences run side by side (a short sequence fills only a few SMs), each with its own slice of the scratch.
// Made once per device; the mutex also keeps two host threads from interleaving their use of the fork event.
namespace {
constexpr int kMaxLanes = 8;
struct LanePool {
  cudaStream_t lane[kMaxLanes];
  cudaEvent_t fork, join[kMaxLanes];
};
std::mutex g_lane_mutex;
LanePool* g_lane_pool[64] = {};
LanePool* lane_pool_locked() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (g_lane_pool[dev]) return g_lane_pool[dev];
  LanePool* lp = new LanePool();
  bool ok = cudaEventCreateWithFlags(&lp->fork, cudaEventDisableTiming) == cudaSuccess;
  for (int i = 0; ok && i < kMaxLanes; ++i)
    ok = cudaStreamCreateWithFlags(&lp->lane[i], cudaStreamNonBlocking) == cudaSuccess &&
         cudaEventCreateWithFlags(&lp->join[i], cudaEventDisableTiming) == cudaSuccess;
  if (!ok) {
    delete lp;  // a device that cannot give a handful of streams: the caller falls back to one lane
    return nullptr;
  }
  return g_lane_pool[dev] = lp;
}
}  // namespace

int kb_sa_bwd_varlen(const kb_sa_varlen_params* p, void* stream) {
  int rc = check_varlen(p, true);
  if (rc || p->B == 0) return rc;
  const int32_t Hk = p->H_kv > 0 ? p->H_kv : p->H, D = p->D;
  const int64_t total = p->cu_seqlens[p->B];
  if (p->lanes > (uint32_t)kMaxLanes) return KB_ERR_BAD_ARGUMENT;
  int32_t max_len = 0;
  for (int32_t b = 0; b < p->B; ++b) max_len = kb_max_i32(max_len, p->cu_seqlens[b + 1] - p->cu_seqlens[b]);
  if (total == 0) return KB_OK;
  if (p->cu_seqlens_dev) {
    // one launch per kernel: the kernels find every sequence's first row and length in the device copy
    kb_sa_bwd_params g = {};
    g.q = packed_view(p->q, 0, p->H, D);
    g.k = packed_view(p->k, 0, Hk, D);
    g.v = packed_view(p->v, 0, Hk, D);
    g.o = packed_view(p->o, 0, p->H, D);
    g.d_o = packed_view(p->d_o, 0, p->H, D);
    g.lse = p->lse;
    g.lse_stride[0] = total * p->H, g.lse_stride[1] = total;
    g.dq = p->dq, g.dk = p->dk, g.dv = p->dv;
    g.dq_stride[0] = total * p->H * D, g.dq_stride[1] = D, g.dq_stride[2] = (int64_t)p->H * D;
    g.dkv_stride[0] = total * Hk * D, g.dkv_stride[1] = D, g.dkv_stride[2] = (int64_t)Hk * D;
    g.delta_ws = p->delta_ws;
    g.ds_ws = p->ds_ws, g.ds_ws_bytes = p->ds_ws_bytes;
    g.B = p->B, g.H = p->H, g.T = max_len, g.D = D, g.H_kv = Hk;
    g.dtype = p->dtype, g.context_size = p->context_size, g.back_contexts = p->back_contexts;
    g.sm_scale = p->sm_scale, g.flags = p->flags & ~KB_FLAG_BWD_TWO_PASS, g.status = p->status;
    g.cu_seqlens = p->cu_seqlens_dev, g.total_rows = (int32_t)total;
    return kb_sa_bwd(&g, stream);
  }
  int lanes = p->lanes > 1 ? (int)p->lanes : 1;
  std::unique_lock<std::mutex> lock(g_lane_mutex, std::defer_lock);
  LanePool* pool = nullptr;
  cudaStream_t caller = static_cast<cudaStream_t>(stream);
  if (lanes > 1) {
    lock.lock();
    pool = lane_pool_locked();
    if (!pool) {
      lanes = 1;
      lock.unlock();
    } else {
      KB_CUDA_TRY(cudaEventRecord(pool->fork, caller));
      for (int i = 0; i < lanes; ++i) KB_CUDA_TRY(cudaStreamWaitEvent(pool->lane[i], pool->fork, 0));
    }
  }
  const uint64_t ds_lane_bytes = (p->ds_ws_bytes / (uint64_t)lanes) & ~(uint64_t)255;
  int32_t live = 0;
  for (int32_t b = 0; b < p->B; ++b) {
    const int64_t r0 = p->cu_seqlens[b];
    const int32_t len = p->cu_seqlens[b + 1] - p->cu_seqlens[b];
    if (len == 0) continue;
    const int lane = live++ % lanes;
    kb_sa_bwd_params g = {};
    g.q = packed_view(p->q, r0, p->H, D);
    g.k = packed_view(p->k, r0, Hk, D);
    g.v = packed_view(p->v, r0, Hk, D);
    g.o = packed_view(p->o, r0, p->H, D);
    g.d_o = packed_view(p->d_o, r0, p->H, D);
    g.lse = p->lse + r0;
    g.lse_stride[0] = total * p->H, g.lse_stride[1] = total;
    g.dq = static_cast<uint16_t*>(p->dq) + r0 * p->H * D;
    g.dq_stride[0] = (int64_t)len * p->H * D, g.dq_stride[1] = D, g.dq_stride[2] = (int64_t)p->H * D;
    g.dk = static_cast<uint16_t*>(p->dk) + r0 * Hk * D;
    g.dv = static_cast<uint16_t*>(p->dv) + r0 * Hk * D;
    g.dkv_stride[0] = (int64_t)len * Hk * D, g.dkv_stride[1] = D, g.dkv_stride[2] = (int64_t)Hk * D;
    g.delta_ws = p->delta_ws + (int64_t)lane * p->H * max_len;
    g.ds_ws = static_cast<uint8_t*>(p->ds_ws) + (uint64_t)lane * ds_lane_bytes, g.ds_ws_bytes = ds_lane_bytes;
    g.B = 1, g.H = p->H, g.T = len, g.D = D, g.H_kv = Hk;
    g.dtype = p->dtype, g.context_size = p->context_size, g.back_contexts = p->back_contexts;
    g.sm_scale = p->sm_scale, g.flags = p->flags & ~KB_FLAG_BWD_TWO_PASS, g.status = p->status;
    rc = kb_sa_bwd(&g, pool ? pool->lane[lane] : caller);
    if (rc) break;
  }
  if (pool) {
    // the caller's stream continues after every lane, also when a launch failed half way
    for (int i = 0; i < lanes; ++i) {
      const bool ok = cudaEventRecord(pool->join[i], pool->lane[i]) == cudaSuccess &&
                      cudaStreamWaitEvent(caller, pool->join[i], 0) == cudaSuccess;
      if (!ok && !rc) rc = KB_ERR_LAUNCH;
    }
  }
  return rc;
}

uint64_t kb_sa_bwd_workspace_bytes(int32_t B, int32_t H, int32_t T, int32_t D, int32_t dtype, int32_t context_size,
                                   int32_t back_contexts) {
#ifdef KB_HAVE_SM100_BWD_FUSED
  if (B > 0 && H > 0 && T > 0 && context_size >= 1 && back_contexts >= 0 && kb::sm100_shape_ok(dtype, D, 0)) {
    const int32_t c = kb_clamp_context(context_size, T);
    return kb::sa_bwd_fused_workspace_bytes(B, H, T, c, kb_clamp_back(back_contexts, T, c));
  }
#endif
  (void)B, (void)H, (void)T, (void)D, (void)dtype, (void)context_size, (void)back_contexts;
  return 0;
}

uint64_t kb_sa_bwd_varlen_workspace_bytes(int32_t B, int32_t H, int32_t total_rows, int32_t max_len, int32_t D,
                                          int32_t dtype, int32_t context_size, int32_t back_contexts) {
#ifdef KB_HAVE_SM100_BWD_FUSED
  if (B > 0 && H > 0 && total_rows > 0 && max_len > 0 && max_len <= total_rows && context_size >= 1 && back_contexts >= 0 &&
      kb::sm100_shape_ok(dtype, D, 0)) {
    const int32_t c = kb_clamp_context(context_size, max_len);
    return kb::sa_bwd_fused_workspace_bytes_packed(B, H, total_rows, max_len, c, kb_clamp_back(back_contexts, max_len, c));
  }
#endif
  (void)B, (void)H, (void)total_rows, (void)max_len, (void)D, (void)dtype, (void)context_size, (void)back_contexts;
  return 0;
}

int kb_softmax_fwd(const kb_softmax_params* p, void* stream) {
  if (!p || p->rows < 0 || p->cols < 0) return KB_ERR_BAD_ARGUMENT;
  if (!kb::dtype_ok(p->dtype)) return KB_ERR_UNSUPPORTED;
  if (p->rows == 0 || p->cols == 0) return KB_OK;
  if (!p->x || !p->y) return KB_ERR_BAD_ARGUMENT;
  return kb::softmax_rows(*p, static_cast<cudaStream_t>(stream));
}

int kb_sa_plan(int32_t T, int32_t seq_len, int32_t context_size, int32_t back_contexts, int32_t tile_q,
               int32_t tile_k, int32_t* fwd_ranges, int32_t* bwd_ranges) {
  if (T < 0 || context_size < 1 || back_contexts < 0 || tile_q < 1 || tile_k < 1) return -KB_ERR_BAD_ARGUMENT;
  const int32_t len = kb_clamp_len(seq_len, T);
  const int32_t c = kb_clamp_context(context_size, T);
  const int32_t back = kb_clamp_back(back_contexts, T, c);
  const int32_t nq = kb_cdiv_i32(T, tile_q), nk = kb_cdiv_i32(T, tile_k);
  if (fwd_ranges)
    for (int32_t i = 0; i < nq; ++i) {
      KbTileRange r = kb_fwd_kv_range(i * tile_q, tile_q, tile_k, len, c, back);
      fwd_ranges[2 * i] = r.begin;
      fwd_ranges[2 * i + 1] = r.end;
    }
  if (bwd_ranges)
    for (int32_t j = 0; j < nk; ++j) {
      KbTileRange r = kb_bwd_q_range(j * tile_k, tile_q, tile_k, len, c, back);
      bwd_ranges[2 * j] = r.begin;
      bwd_ranges[2 * j + 1] = r.end;
    }
  return nq;
}

int kb_sa_tile_config(int32_t dtype, int32_t D, int32_t context_size, uint32_t flags, int32_t unit_inner_stride,
                      int32_t which, int32_t* path, int32_t* tile_q, int32_t* tile_k, int32_t* stages) {
  namespace t = kb::tiles;
  // One row per (dtype, head dim) class today: the measurements behind the table (profiles/) found no
  // chunk length for which another tile beats 128-row tiles on the tcgen05 path, so `context_size` does
  // not select a row; it stays in the signature because the table is keyed on it.
  if (context_size < 1) return KB_ERR_BAD_ARGUMENT;
  if (!kb::dtype_ok(dtype) || !kb::head_dim_ok(D)) return KB_ERR_UNSUPPORTED;
  if (which < 0 || which > 4) return KB_ERR_BAD_ARGUMENT;
  int32_t pth = KB_PATH_GENERIC, tq = t::generic_tile(D), tk = tq, st = t::kGenericStages;
#ifdef KB_HAVE_SM100
  if (kb::sm100_shape_ok(dtype, D, flags) && unit_inner_stride) {
    // every number below is the constant the kernel itself is compiled with (tiles.h)
    if (which == 0) {
      pth = KB_PATH_SM100;
      tq = t::kFwdQRows * t::kFwdQTiles;
      tk = t::kFwdKeys;
      st = t::kFwdStagesK;  // K ring; the V ring has t::kFwdStagesV stages
    }
#ifdef KB_HAVE_SM100_BWD
    if (which == 1 || which == 2) {
      pth = KB_PATH_SM100;
      tq = which == 1 ? t::kTwoPassStationary : t::kTwoPassStreamed;
      tk = which == 1 ? t::kTwoPassStreamed : t::kTwoPassStationary;
      st = t::kTwoPassStagesFirst;  // ring of the first streamed operand; the second has kTwoPassStagesSecond
    }
#endif
#ifdef KB_HAVE_SM100_BWD_FUSED
    if (which == 3) {
      pth = KB_PATH_SM100;
      tq = t::kMainQueries;
      tk = t::kMainKeys;
      st = t::kMainStagesQ;
    }
    if (which == 4) {
      pth = KB_PATH_SM100;
      tq = t::kDqQueries;
      tk = t::kDqKeys;
      st = t::kDqStages;
    }
#endif
  }
#else
  (void)flags;
  (void)unit_inner_stride;
#endif
  if (path) *path = pth;
  if (tile_q) *tile_q = tq;
  if (tile_k) *tile_k = tk;
  if (stages) *stages = st;
  return KB_OK;
}

int64_t kb_launch_count(void) { return kb::g_launches.load(std::memory_order_relaxed); }

const char* kb_strerror(int status) {
  switch (status) {
    case KB_OK: return "ok";
    case KB_ERR_BAD_ARGUMENT: return "bad argument (null pointer, negative size, context_size < 1 or back_contexts < 0)";
    case KB_ERR_UNSUPPORTED: return "unsupported dtype / head_dim (need fp32, fp16 or bf16 and D in {16,32,64,128,256})";
    case KB_ERR_LAUNCH: return "CUDA launch failed (see kb_last_cuda_error)";
    case KB_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case KB_ERR_TOO_LARGE: return "problem too large for this entry point";
    default: return "unknown status";
  }
}

const char* kb_last_cuda_error(void) { return kb::g_cuda_error; }

const char* kb_version(void) { return "kernels_b200 0.1 (sm_100a)"; }

}  // extern "C"
