// extern "C" surface of the library (declared in include/kernels_b200.h): argument
// validation, kernel-family selection and the host-side schedule planner.
#include <atomic>
#include <cstdio>
#include <cstring>

#include "common.cuh"

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

int run_fwd(const kb_sa_fwd_params* p, void* stream, bool dense) {
  int rc = check_common(p);
  if (rc) return rc;
  if (kv_heads(p) < 0) return KB_ERR_BAD_ARGUMENT;
  if (!dense && (p->context_size < 1 || p->back_contexts < 0)) return KB_ERR_BAD_ARGUMENT;
  if (empty(p->B, p->H, p->T)) return KB_OK;
  if (!p->q.data || !p->k.data || !p->v.data || !p->o) return KB_ERR_BAD_ARGUMENT;
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
  if (kv_heads(p) != p->H) return KB_ERR_UNSUPPORTED;  // the generic kernels want one K/V head per query head
  return sa_fwd_generic(*p, c, back, s);
}

}  // namespace
}  // namespace kb

extern "C" {

int kb_sa_fwd(const kb_sa_fwd_params* p, void* stream) { return kb::run_fwd(p, stream, /*dense=*/false); }

int kb_fa_fwd(const kb_sa_fwd_params* p, void* stream) { return kb::run_fwd(p, stream, /*dense=*/true); }

int kb_sa_bwd(const kb_sa_bwd_params* p, void* stream) {
  int rc = kb::check_common(p);
  if (rc) return rc;
  if (p->context_size < 1 || p->back_contexts < 0 || kb::kv_heads(p) < 0) return KB_ERR_BAD_ARGUMENT;
  if (kb::empty(p->B, p->H, p->T)) return KB_OK;
  if (!p->q.data || !p->k.data || !p->v.data || !p->o.data || !p->d_o.data || !p->lse || !p->dq || !p->dk ||
      !p->dv || !p->delta_ws)
    return KB_ERR_BAD_ARGUMENT;
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
    if (kb::kv_heads(p) != p->H) return KB_ERR_UNSUPPORTED;  // shared K/V heads: single-evaluation kernels only
    const int rc = kb::sa_bwd_sm100(*p, c, back, s);
    if (rc != KB_ERR_UNSUPPORTED) return rc;
  }
#endif
  if (kb::kv_heads(p) != p->H) return KB_ERR_UNSUPPORTED;
  return kb::sa_bwd_generic(*p, c, back, s);
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
  (void)context_size;
  if (!kb::dtype_ok(dtype) || !kb::head_dim_ok(D)) return KB_ERR_UNSUPPORTED;
  if (which < 0 || which > 4) return KB_ERR_BAD_ARGUMENT;
  int32_t pth = KB_PATH_GENERIC, tq = D <= 128 ? 64 : 32, tk = tq, st = 1;
#ifdef KB_HAVE_SM100
  if (kb::sm100_shape_ok(dtype, D, flags) && unit_inner_stride) {
    // forward: two 128-row q tiles per CTA share 128-key K/V tiles (K ring 3 deep, V ring 2 deep);
    // backward passes: 128 stationary rows, 128-row streamed tiles (rings 3 and 2 deep)
    if (which == 0) {
      pth = KB_PATH_SM100;
      tq = 256;
      tk = 128;
      st = 3;
    }
#ifdef KB_HAVE_SM100_BWD
    if (which == 1 || which == 2) {
      pth = KB_PATH_SM100;
      tq = 128;
      tk = 128;
      st = 3;
    }
#endif
#ifdef KB_HAVE_SM100_BWD_FUSED
    // single-evaluation backward: main kernel (Q ring 2 deep), dQ kernel (dS / K ring 3 deep)
    if (which == 3 || which == 4) {
      pth = KB_PATH_SM100;
      tq = 128;
      tk = 128;
      st = which == 3 ? 2 : 3;
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
