// Shared helpers of the library's translation units: dtype conversion, error plumbing and
// the launch counter.  Nothing here is part of the exported ABI.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kernels_b200.h"
#include "schedule.h"

namespace kb {

constexpr float kLog2e = 1.4426950408889634f;

// ---- host-side error state -------------------------------------------------------------
void set_cuda_error(cudaError_t e, const char* where);  // defined in capi.cu
void count_launch(int n = 1);                           // defined in capi.cu

#define KB_CUDA_TRY(expr)                          \
  do {                                             \
    cudaError_t _e = (expr);                       \
    if (_e != cudaSuccess) {                       \
      ::kb::set_cuda_error(_e, #expr);             \
      return KB_ERR_LAUNCH;                        \
    }                                              \
  } while (0)

// Call after a <<<>>> launch: records the launch, maps a launch error to KB_ERR_LAUNCH.
#define KB_LAUNCH_CHECK(what)                      \
  do {                                             \
    ::kb::count_launch();                          \
    cudaError_t _e = cudaGetLastError();           \
    if (_e != cudaSuccess) {                       \
      ::kb::set_cuda_error(_e, what);              \
      return KB_ERR_LAUNCH;                        \
    }                                              \
  } while (0)

// ---- element conversion ----------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Problem description shared by the kernel launchers (dense == single chunk, no look-back).
struct AttnShape {
  int32_t B, H, T, D;
  int32_t c, back;
  float scale_log2;  // sm_scale * log2(e)
  float sm_scale;
};

// ---- launchers implemented in the kernel translation units -----------------------------
int sa_fwd_generic(const kb_sa_fwd_params& p, int32_t c, int32_t back, cudaStream_t s);
int sa_bwd_generic(const kb_sa_bwd_params& p, int32_t c, int32_t back, cudaStream_t s);
int sa_fwd_sm100(const kb_sa_fwd_params& p, int32_t c, int32_t back, cudaStream_t s);
int sa_fwd_sm100_fp8(const kb_sa_fwd_fp8_params& p, int32_t c, int32_t back, cudaStream_t s);
int sa_bwd_sm100(const kb_sa_bwd_params& p, int32_t c, int32_t back, cudaStream_t s);
int sa_bwd_fused_sm100(const kb_sa_bwd_params& p, int32_t c, int32_t back, cudaStream_t s);
size_t sa_bwd_fused_workspace_bytes(int32_t B, int32_t H, int32_t T, int32_t c, int32_t back);
size_t sa_bwd_fused_workspace_bytes_packed(int32_t B, int32_t H, int32_t total, int32_t max_len, int32_t c, int32_t back);
int softmax_rows(const kb_softmax_params& p, cudaStream_t s);

}  // namespace kb
