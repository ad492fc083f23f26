// Row softmax  y = exp(x - max) / sum  over the last axis of a [rows, cols] matrix.
//
// HBM-bound: every element is read once and written once (2 * rows * cols * elsize bytes),
// so the kernel keeps a whole row in registers between the reduction and the store and
// moves data in 16-byte vectors with streaming cache hints.
//   * cols <= 32 * 16-byte vectors * 8 : one warp per row, several rows per CTA;
//   * cols <= 256 threads * 16 vectors  : one CTA per row, block reduction through smem;
//   * otherwise, or when rows are not 16-byte aligned: a three-pass scalar kernel.
// Reference semantics: src/softmax/kernel.py:27-91 (natural exponent, fp32 math).
#include <math.h>

#include "common.cuh"

namespace kb {
namespace {

template <typename T>
struct Vec16 {
  static constexpr int kElems = 16 / sizeof(T);
};

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float (&out)[Vec16<T>::kElems]) {
  const int4 raw = __ldcs(reinterpret_cast<const int4*>(p));
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec16<T>::kElems; ++i) out[i] = to_f32(e[i]);
}

template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float (&in)[Vec16<T>::kElems]) {
  int4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec16<T>::kElems; ++i) e[i] = from_f32<T>(in[i]);
  __stcs(reinterpret_cast<int4*>(p), raw);
}

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// One row per GROUP threads (GROUP = 32: warp per row; GROUP = blockDim: CTA per row).
// Each thread holds NV 16-byte vectors of its row; vector v of thread t covers elements
// (v * GROUP + t) * kElems .. +kElems, so a warp's accesses are contiguous.
template <typename T, int NV, int GROUP, int THREADS>
__global__ void __launch_bounds__(THREADS) softmax_rows_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                               int64_t rows, int cols, int64_t xs, int64_t ys) {
  constexpr int E = Vec16<T>::kElems;
  constexpr int ROWS_PER_CTA = THREADS / GROUP;
  __shared__ float red[THREADS / 32];
  const int lane_in_group = threadIdx.x % GROUP;
  const int64_t row = (int64_t)blockIdx.x * ROWS_PER_CTA + threadIdx.x / GROUP;
  const bool row_ok = row < rows;
  const T* xr = x + (row_ok ? row : 0) * xs;
  T* yr = y + (row_ok ? row : 0) * ys;

  float v[NV][E];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (i * GROUP + lane_in_group) * E;
    if (row_ok && col < cols) {
      load_vec<T>(xr + col, v[i]);
    } else {
#pragma unroll
      for (int e = 0; e < E; ++e) v[i][e] = -INFINITY;
    }
#pragma unroll
    for (int e = 0; e < E; ++e) mx = fmaxf(mx, v[i][e]);
  }
  mx = warp_max(mx);
  if (GROUP > 32) {
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < THREADS / 32; ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
  }
  const float mx_l2 = mx * kLog2e;
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int e = 0; e < E; ++e) {
      v[i][e] = exp2f(fmaf(v[i][e], kLog2e, -mx_l2));
      sum += v[i][e];
    }
  sum = warp_sum(sum);
  if (GROUP > 32) {
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    sum = 0.f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) sum += red[w];
  }
  const float inv = 1.f / sum;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (i * GROUP + lane_in_group) * E;
    if (row_ok && col < cols) {
#pragma unroll
      for (int e = 0; e < E; ++e) v[i][e] *= inv;
      store_vec<T>(yr + col, v[i]);
    }
  }
}

// Any shape / alignment: one CTA per row, three passes over the row (max, sum, write).
template <typename T>
__global__ void __launch_bounds__(256) softmax_rows_scalar_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                                  int64_t cols, int64_t xs, int64_t ys) {
  __shared__ float red[8];
  const T* xr = x + (int64_t)blockIdx.x * xs;
  T* yr = y + (int64_t)blockIdx.x * ys;
  float mx = -INFINITY;
  for (int64_t i = threadIdx.x; i < cols; i += 256) mx = fmaxf(mx, to_f32(xr[i]));
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
  for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
  __syncthreads();
  float sum = 0.f;
  for (int64_t i = threadIdx.x; i < cols; i += 256) sum += expf(to_f32(xr[i]) - mx);
  sum = warp_sum(sum);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
  __syncthreads();
  sum = 0.f;
  for (int w = 0; w < 8; ++w) sum += red[w];
  const float inv = 1.f / sum;
  for (int64_t i = threadIdx.x; i < cols; i += 256) yr[i] = from_f32<T>(expf(to_f32(xr[i]) - mx) * inv);
}

template <typename T, int NV, int GROUP, int THREADS>
int launch_vec(const kb_softmax_params& p, cudaStream_t s) {
  constexpr int rows_per_cta = THREADS / GROUP;
  const int64_t ctas = (p.rows + rows_per_cta - 1) / rows_per_cta;
  softmax_rows_kernel<T, NV, GROUP, THREADS><<<(unsigned)ctas, THREADS, 0, s>>>(
      static_cast<const T*>(p.x), static_cast<T*>(p.y), p.rows, (int)p.cols, p.x_row_stride, p.y_row_stride);
  KB_LAUNCH_CHECK("softmax_rows_kernel");
  return KB_OK;
}

template <typename T>
int softmax_typed(const kb_softmax_params& p, cudaStream_t s) {
  constexpr int E = Vec16<T>::kElems;
  const bool aligned = (reinterpret_cast<uintptr_t>(p.x) % 16 == 0) && (reinterpret_cast<uintptr_t>(p.y) % 16 == 0) &&
                       (p.x_row_stride % E == 0) && (p.y_row_stride % E == 0) && (p.cols % E == 0);
  const int64_t vecs = p.cols / E;
  if (aligned && p.rows < (int64_t)1 << 31) {
    if (vecs <= 32 * 1) return launch_vec<T, 1, 32, 256>(p, s);
    if (vecs <= 32 * 2) return launch_vec<T, 2, 32, 256>(p, s);
    if (vecs <= 32 * 4) return launch_vec<T, 4, 32, 256>(p, s);
    if (vecs <= 32 * 8) return launch_vec<T, 8, 32, 256>(p, s);
    if (vecs <= 256 * 2) return launch_vec<T, 2, 256, 256>(p, s);
    if (vecs <= 256 * 4) return launch_vec<T, 4, 256, 256>(p, s);
    if (vecs <= 256 * 8) return launch_vec<T, 8, 256, 256>(p, s);
    if (vecs <= 512 * 8) return launch_vec<T, 8, 512, 512>(p, s);
  }
  if (p.rows >= (int64_t)1 << 31) return KB_ERR_TOO_LARGE;
  softmax_rows_scalar_kernel<T><<<(unsigned)p.rows, 256, 0, s>>>(static_cast<const T*>(p.x), static_cast<T*>(p.y),
                                                                p.cols, p.x_row_stride, p.y_row_stride);
  KB_LAUNCH_CHECK("softmax_rows_scalar_kernel");
  return KB_OK;
}

}  // namespace

int softmax_rows(const kb_softmax_params& p, cudaStream_t s) {
  if (p.rows == 0 || p.cols == 0) return KB_OK;
  switch (p.dtype) {
    case KB_F32: return softmax_typed<float>(p, s);
    case KB_F16: return softmax_typed<__half>(p, s);
    case KB_BF16: return softmax_typed<__nv_bfloat16>(p, s);
    default: return KB_ERR_UNSUPPORTED;
  }
}

}  // namespace kb
