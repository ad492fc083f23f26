// Generic CUDA-core path of streaming attention (forward, dQ pass, dK/dV pass).
//
// Covers every case the reference accepts: fp32/fp16/bf16, head_dim 16..256, arbitrary
// element strides on every input, any context size (non powers of two, larger than T) and
// any look-back.  All arithmetic is IEEE fp32 (the reference's precision="ieee" for fp32
// inputs forbids TF32).  The fp16/bf16 hot shapes are served by the tcgen05 kernels; this
// file is what runs everywhere else.
//
// Work split: one CTA of 256 threads owns one tile of BM query rows (forward, dQ) or BN key
// rows (dK/dV) of one (batch, head) and walks only the live tiles of the streaming schedule
// (schedule.h).  Threads form a 16x16 grid: thread (ty, tx) owns rows ty+16*i and columns
// tx+16*j of every [rows x cols] product, so row reductions are 16-lane shuffles.
//
// Reference semantics followed: src/streaming_attention/kernel.py:205-430 (forward),
// 639-773 and 941-1023 (dQ), 777-937 and 1027-1129 (dK/dV), 453-514 (delta).
#include <math.h>

#include "common.cuh"
#include "sm100_host.h"
#include "tiles.h"

namespace kb {
namespace {

constexpr int kThreads = 256;
constexpr int kPad = 4;  // floats of row padding: keeps float4 alignment, spreads banks

template <typename T>
struct TensorArg {
  const T* p;
  int64_t sb, sh, st, sd;
};

template <typename T>
TensorArg<T> make_arg(const kb_tensor4& t) {
  return TensorArg<T>{static_cast<const T*>(t.data), t.stride[0], t.stride[1], t.stride[2], t.stride[3]};
}

template <typename T>
struct FwdArgs {
  TensorArg<T> q, k, v;
  T* o;
  float* lse;
  const int32_t* lens;
  int64_t lens_stride;
  int32_t H, T_, c, back;
  float scale_log2;
};

template <typename T>
struct BwdArgs {
  TensorArg<T> q, k, v, o, d_o;
  const float* lse;
  T* dq;
  T* dk;
  T* dv;
  float* delta;
  const int32_t* lens;
  int64_t lens_stride;
  int32_t H, T_, c, back;
  float scale_log2, sm_scale;
};

// [ROWS x D] tile of one (b, h) slice -> shared memory as fp32; rows past T read as zero.
template <int D, int ROWS, typename T>
__device__ __forceinline__ void load_tile(float* dst, const T* slice, int64_t st, int64_t sd, int row0, int T_) {
  constexpr int LD = D + kPad;
  for (int idx = threadIdx.x; idx < ROWS * D; idx += kThreads) {
    int r = idx / D, d = idx - r * D;
    int t = row0 + r;
    float x = 0.f;
    if (t < T_) x = to_f32(slice[(int64_t)t * st + (int64_t)d * sd]);
    dst[r * LD + d] = x;
  }
}

// acc[i][j] = sum_d A[ty+16i][d] * Bm[tx+16j][d]
template <int D, int RM, int RN>
__device__ __forceinline__ void tile_abt(const float* A, const float* Bm, float (&acc)[RM][RN], int ty, int tx) {
  constexpr int LD = D + kPad;
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int j = 0; j < RN; ++j) acc[i][j] = 0.f;
#pragma unroll 4
  for (int d = 0; d < D; d += 4) {
    float4 a[RM], b[RN];
#pragma unroll
    for (int i = 0; i < RM; ++i) a[i] = *reinterpret_cast<const float4*>(&A[(ty + 16 * i) * LD + d]);
#pragma unroll
    for (int j = 0; j < RN; ++j) b[j] = *reinterpret_cast<const float4*>(&Bm[(tx + 16 * j) * LD + d]);
#pragma unroll
    for (int i = 0; i < RM; ++i)
#pragma unroll
      for (int j = 0; j < RN; ++j) {
        acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
        acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
        acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
        acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
      }
  }
}

__device__ __forceinline__ float half_warp_max(float x) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float half_warp_sum(float x) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

__device__ __forceinline__ int load_len(const int32_t* lens, int64_t stride, int b, int T_) {
  return lens ? kb_clamp_len(lens[(int64_t)b * stride], T_) : T_;
}

// ------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------
template <int D, int BM, int BN, typename T>
__global__ void __launch_bounds__(kThreads) sa_fwd_generic_kernel(FwdArgs<T> a) {
  constexpr int LD = D + kPad, RM = BM / 16, RN = BN / 16, DV = D / 16, PLD = BN + 1;
  extern __shared__ __align__(16) float smem[];
  float* Qs = smem;
  float* Ks = Qs + BM * LD;
  float* Vs = Ks + BN * LD;
  float* Ps = Vs + BN * LD;

  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * BM;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int T_ = a.T_, c = a.c, back = a.back;
  const int len = load_len(a.lens, a.lens_stride, b, T_);
  T* o_slice = a.o + ((int64_t)b * a.H + h) * T_ * D;
  float* lse_slice = a.lse ? a.lse + ((int64_t)b * a.H + h) * T_ : nullptr;

  const KbTileRange kr = kb_fwd_kv_range(q0, BM, BN, len, c, back);

  float m[RM], l[RM], acc[RM][DV];
  int qchunk[RM];
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
    qchunk[i] = (q0 + ty + 16 * i) / c;
#pragma unroll
    for (int dv = 0; dv < DV; ++dv) acc[i][dv] = 0.f;
  }

  if (kr.begin < kr.end) {
    load_tile<D, BM>(Qs, a.q.p + b * a.q.sb + h * a.q.sh, a.q.st, a.q.sd, q0, T_);
    const T* k_slice = a.k.p + b * a.k.sb + h * a.k.sh;
    const T* v_slice = a.v.p + b * a.v.sb + h * a.v.sh;
    for (int kt = kr.begin; kt < kr.end; ++kt) {
      const int k0 = kt * BN;
      __syncthreads();
      load_tile<D, BN>(Ks, k_slice, a.k.st, a.k.sd, k0, T_);
      load_tile<D, BN>(Vs, v_slice, a.v.st, a.v.sd, k0, T_);
      __syncthreads();

      float s[RM][RN];
      tile_abt<D, RM, RN>(Qs, Ks, s, ty, tx);

      int kchunk[RN];
#pragma unroll
      for (int j = 0; j < RN; ++j) kchunk[j] = (k0 + tx + 16 * j) / c;

#pragma unroll
      for (int i = 0; i < RM; ++i) {
        const int qi = q0 + ty + 16 * i;
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < RN; ++j) {
          const bool live = kb_live(qi, k0 + tx + 16 * j, qchunk[i], kchunk[j], len, back);
          s[i][j] = live ? s[i][j] * a.scale_log2 : -INFINITY;
          mx = fmaxf(mx, s[i][j]);
        }
        mx = half_warp_max(mx);
        const float m_new = fmaxf(m[i], mx);
        const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = exp2f(m[i] - m_safe);
        float rs = 0.f;
#pragma unroll
        for (int j = 0; j < RN; ++j) {
          const float p = exp2f(s[i][j] - m_safe);
          Ps[(ty + 16 * i) * PLD + tx + 16 * j] = p;
          rs += p;
        }
        rs = half_warp_sum(rs);
        l[i] = l[i] * alpha + rs;
        m[i] = m_new;
#pragma unroll
        for (int dv = 0; dv < DV; ++dv) acc[i][dv] *= alpha;
      }
      __syncthreads();

#pragma unroll 4
      for (int kk = 0; kk < BN; ++kk) {
        float pv[RM];
#pragma unroll
        for (int i = 0; i < RM; ++i) pv[i] = Ps[(ty + 16 * i) * PLD + kk];
#pragma unroll
        for (int dv = 0; dv < DV; ++dv) {
          const float vv = Vs[kk * LD + tx + 16 * dv];
#pragma unroll
          for (int i = 0; i < RM; ++i) acc[i][dv] = fmaf(pv[i], vv, acc[i][dv]);
        }
      }
    }
  }

#pragma unroll
  for (int i = 0; i < RM; ++i) {
    const int r = q0 + ty + 16 * i;
    if (r >= T_) continue;
    const bool valid = r < len;
    const float inv = valid ? 1.f / l[i] : 0.f;
#pragma unroll
    for (int dv = 0; dv < DV; ++dv) o_slice[(int64_t)r * D + tx + 16 * dv] = from_f32<T>(valid ? acc[i][dv] * inv : 0.f);
    if (lse_slice && tx == 0) lse_slice[r] = valid ? m[i] + log2f(l[i]) : 0.f;
  }
}

// ------------------------------------------------------------------------------------------
// backward, dQ pass (also produces delta = rowsum(O * dO))
// ------------------------------------------------------------------------------------------
template <int D, int BM, int BN, typename T>
__global__ void __launch_bounds__(kThreads) sa_bwd_dq_generic_kernel(BwdArgs<T> a) {
  constexpr int LD = D + kPad, RM = BM / 16, RN = BN / 16, DV = D / 16, PLD = BN + 1;
  extern __shared__ __align__(16) float smem[];
  float* Qs = smem;
  float* dOs = Qs + BM * LD;
  float* Ks = dOs + BM * LD;
  float* Vs = Ks + BN * LD;
  float* dSs = Vs + BN * LD;

  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * BM;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int T_ = a.T_, c = a.c, back = a.back;
  const int len = load_len(a.lens, a.lens_stride, b, T_);
  const int64_t bh = (int64_t)b * a.H + h;
  T* dq_slice = a.dq + bh * T_ * D;
  float* delta_slice = a.delta + bh * T_;
  const float* lse_slice = a.lse + bh * T_;

  const KbTileRange kr = kb_fwd_kv_range(q0, BM, BN, len, c, back);

  float acc[RM][DV], delta[RM], lse[RM];
  int qchunk[RM];
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    delta[i] = 0.f;
    lse[i] = 0.f;
    qchunk[i] = (q0 + ty + 16 * i) / c;
#pragma unroll
    for (int dv = 0; dv < DV; ++dv) acc[i][dv] = 0.f;
  }

  if (kr.begin < kr.end) {
    load_tile<D, BM>(Qs, a.q.p + b * a.q.sb + h * a.q.sh, a.q.st, a.q.sd, q0, T_);
    load_tile<D, BM>(dOs, a.d_o.p + b * a.d_o.sb + h * a.d_o.sh, a.d_o.st, a.d_o.sd, q0, T_);
    __syncthreads();
    const T* o_slice = a.o.p + b * a.o.sb + h * a.o.sh;
#pragma unroll
    for (int i = 0; i < RM; ++i) {
      const int r = q0 + ty + 16 * i;
      float part = 0.f;
      if (r < len) {
#pragma unroll
        for (int dv = 0; dv < DV; ++dv) {
          const int d = tx + 16 * dv;
          part = fmaf(to_f32(o_slice[(int64_t)r * a.o.st + (int64_t)d * a.o.sd]), dOs[(ty + 16 * i) * LD + d], part);
        }
      }
      delta[i] = half_warp_sum(part);
      if (r < len) lse[i] = lse_slice[r];
    }

    const T* k_slice = a.k.p + b * a.k.sb + h * a.k.sh;
    const T* v_slice = a.v.p + b * a.v.sb + h * a.v.sh;
    for (int kt = kr.begin; kt < kr.end; ++kt) {
      const int k0 = kt * BN;
      __syncthreads();
      load_tile<D, BN>(Ks, k_slice, a.k.st, a.k.sd, k0, T_);
      load_tile<D, BN>(Vs, v_slice, a.v.st, a.v.sd, k0, T_);
      __syncthreads();

      float s[RM][RN], dp[RM][RN];
      tile_abt<D, RM, RN>(Qs, Ks, s, ty, tx);
      tile_abt<D, RM, RN>(dOs, Vs, dp, ty, tx);
#pragma unroll
      for (int j = 0; j < RN; ++j) {
        const int kj = k0 + tx + 16 * j;
        const int kchunk = kj / c;
#pragma unroll
        for (int i = 0; i < RM; ++i) {
          const bool live = kb_live(q0 + ty + 16 * i, kj, qchunk[i], kchunk, len, back);
          float ds = 0.f;
          if (live) {
            const float p = exp2f(s[i][j] * a.scale_log2 - lse[i]);
            ds = p * (dp[i][j] - delta[i]);
          }
          dSs[(ty + 16 * i) * PLD + tx + 16 * j] = ds;
        }
      }
      __syncthreads();
#pragma unroll 4
      for (int kk = 0; kk < BN; ++kk) {
        float dsv[RM];
#pragma unroll
        for (int i = 0; i < RM; ++i) dsv[i] = dSs[(ty + 16 * i) * PLD + kk];
#pragma unroll
        for (int dv = 0; dv < DV; ++dv) {
          const float kv = Ks[kk * LD + tx + 16 * dv];
#pragma unroll
          for (int i = 0; i < RM; ++i) acc[i][dv] = fmaf(dsv[i], kv, acc[i][dv]);
        }
      }
    }
  }

#pragma unroll
  for (int i = 0; i < RM; ++i) {
    const int r = q0 + ty + 16 * i;
    if (r >= T_) continue;
#pragma unroll
    for (int dv = 0; dv < DV; ++dv) dq_slice[(int64_t)r * D + tx + 16 * dv] = from_f32<T>(acc[i][dv] * a.sm_scale);
    if (tx == 0) delta_slice[r] = delta[i];
  }
}

// ------------------------------------------------------------------------------------------
// backward, dK/dV pass (reads delta written by the dQ pass)
// ------------------------------------------------------------------------------------------
template <int D, int BM, int BN, typename T>
__global__ void __launch_bounds__(kThreads) sa_bwd_dkdv_generic_kernel(BwdArgs<T> a) {
  constexpr int LD = D + kPad, RM = BM / 16, RN = BN / 16, DV = D / 16, PLD = BN + 1;
  extern __shared__ __align__(16) float smem[];
  float* Qs = smem;
  float* dOs = Qs + BM * LD;
  float* Ks = dOs + BM * LD;
  float* Vs = Ks + BN * LD;
  float* Ps = Vs + BN * LD;
  float* dSs = Ps + BM * PLD;
  float* lse_s = dSs + BM * PLD;
  float* delta_s = lse_s + BM;

  const int b = blockIdx.z, h = blockIdx.y, k0 = blockIdx.x * BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int T_ = a.T_, c = a.c, back = a.back;
  const int len = load_len(a.lens, a.lens_stride, b, T_);
  const int64_t bh = (int64_t)b * a.H + h;
  T* dk_slice = a.dk + bh * T_ * D;
  T* dv_slice = a.dv + bh * T_ * D;
  const float* delta_slice = a.delta + bh * T_;
  const float* lse_slice = a.lse + bh * T_;

  const KbTileRange qr = kb_bwd_q_range(k0, BM, BN, len, c, back);

  float acc_dk[RN][DV], acc_dv[RN][DV];
  int kchunk[RN];
#pragma unroll
  for (int j = 0; j < RN; ++j) {
    kchunk[j] = (k0 + tx + 16 * j) / c;
#pragma unroll
    for (int dv = 0; dv < DV; ++dv) acc_dk[j][dv] = acc_dv[j][dv] = 0.f;
  }

  if (qr.begin < qr.end) {
    load_tile<D, BN>(Ks, a.k.p + b * a.k.sb + h * a.k.sh, a.k.st, a.k.sd, k0, T_);
    load_tile<D, BN>(Vs, a.v.p + b * a.v.sb + h * a.v.sh, a.v.st, a.v.sd, k0, T_);
    const T* q_slice = a.q.p + b * a.q.sb + h * a.q.sh;
    const T* do_slice = a.d_o.p + b * a.d_o.sb + h * a.d_o.sh;
    for (int qt = qr.begin; qt < qr.end; ++qt) {
      const int q0 = qt * BM;
      __syncthreads();
      load_tile<D, BM>(Qs, q_slice, a.q.st, a.q.sd, q0, T_);
      load_tile<D, BM>(dOs, do_slice, a.d_o.st, a.d_o.sd, q0, T_);
      if (threadIdx.x < BM) {
        const int r = q0 + threadIdx.x;
        lse_s[threadIdx.x] = r < len ? lse_slice[r] : 0.f;
        delta_s[threadIdx.x] = r < len ? delta_slice[r] : 0.f;
      }
      __syncthreads();

      float s[RM][RN], dp[RM][RN];
      tile_abt<D, RM, RN>(Qs, Ks, s, ty, tx);
      tile_abt<D, RM, RN>(dOs, Vs, dp, ty, tx);
#pragma unroll
      for (int i = 0; i < RM; ++i) {
        const int ri = ty + 16 * i;
        const int qi = q0 + ri;
        const int qchunk = qi / c;
        const float lse = lse_s[ri], delta = delta_s[ri];
#pragma unroll
        for (int j = 0; j < RN; ++j) {
          const bool live = kb_live(qi, k0 + tx + 16 * j, qchunk, kchunk[j], len, back);
          float p = 0.f, ds = 0.f;
          if (live) {
            p = exp2f(s[i][j] * a.scale_log2 - lse);
            ds = p * (dp[i][j] - delta);
          }
          Ps[ri * PLD + tx + 16 * j] = p;
          dSs[ri * PLD + tx + 16 * j] = ds;
        }
      }
      __syncthreads();
      // thread (ty, tx) now owns key rows ty+16j and head-dim columns tx+16dv
#pragma unroll 2
      for (int qq = 0; qq < BM; ++qq) {
        float pk[RN], dsk[RN];
#pragma unroll
        for (int j = 0; j < RN; ++j) {
          pk[j] = Ps[qq * PLD + ty + 16 * j];
          dsk[j] = dSs[qq * PLD + ty + 16 * j];
        }
#pragma unroll
        for (int dv = 0; dv < DV; ++dv) {
          const float dov = dOs[qq * LD + tx + 16 * dv];
          const float qv = Qs[qq * LD + tx + 16 * dv];
#pragma unroll
          for (int j = 0; j < RN; ++j) {
            acc_dv[j][dv] = fmaf(pk[j], dov, acc_dv[j][dv]);
            acc_dk[j][dv] = fmaf(dsk[j], qv, acc_dk[j][dv]);
          }
        }
      }
    }
  }

#pragma unroll
  for (int j = 0; j < RN; ++j) {
    const int r = k0 + ty + 16 * j;
    if (r >= T_) continue;
#pragma unroll
    for (int dv = 0; dv < DV; ++dv) {
      dk_slice[(int64_t)r * D + tx + 16 * dv] = from_f32<T>(acc_dk[j][dv] * a.sm_scale);
      dv_slice[(int64_t)r * D + tx + 16 * dv] = from_f32<T>(acc_dv[j][dv]);
    }
  }
}

// ------------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------------
template <int D, typename T>
int launch_fwd(const kb_sa_fwd_params& p, int32_t c, int32_t back, cudaStream_t s) {
  constexpr int BM = tiles::generic_tile(D), BN = BM;
  constexpr int LD = D + kPad;
  constexpr size_t smem = sizeof(float) * (size_t)(BM * LD + 2 * BN * LD + BM * (BN + 1));
  auto kern = sa_fwd_generic_kernel<D, BM, BN, T>;
  int dev = 0, n_sm = 0;
  if (!device_sm_count(&dev, &n_sm)) return KB_ERR_LAUNCH;
  static std::atomic<bool> smem_opted_in[kMaxDevices];
  KB_CUDA_TRY(opt_in_smem_once(kern, smem, dev, smem_opted_in));
  FwdArgs<T> a;
  a.q = make_arg<T>(p.q);
  a.k = make_arg<T>(p.k);
  a.v = make_arg<T>(p.v);
  a.o = static_cast<T*>(p.o);
  a.lse = p.lse;
  a.lens = p.lens;
  a.lens_stride = p.lens_stride;
  a.H = p.H;
  a.T_ = p.T;
  a.c = c;
  a.back = back;
  a.scale_log2 = p.sm_scale * kLog2e;
  dim3 grid(kb_cdiv_i32(p.T, BM), p.H, p.B);
  kern<<<grid, kThreads, smem, s>>>(a);
  KB_LAUNCH_CHECK("sa_fwd_generic_kernel");
  return KB_OK;
}

template <int D, typename T>
int launch_bwd(const kb_sa_bwd_params& p, int32_t c, int32_t back, cudaStream_t s) {
  constexpr int BM = tiles::generic_tile(D), BN = BM;
  constexpr int LD = D + kPad;
  constexpr size_t smem_dq = sizeof(float) * (size_t)(2 * BM * LD + 2 * BN * LD + BM * (BN + 1));
  constexpr size_t smem_dkdv = sizeof(float) * (size_t)(2 * BM * LD + 2 * BN * LD + 2 * BM * (BN + 1) + 2 * BM);
  auto kern_dq = sa_bwd_dq_generic_kernel<D, BM, BN, T>;
  auto kern_dkdv = sa_bwd_dkdv_generic_kernel<D, BM, BN, T>;
  int dev = 0, n_sm = 0;
  if (!device_sm_count(&dev, &n_sm)) return KB_ERR_LAUNCH;
  static std::atomic<bool> dq_opted_in[kMaxDevices], dkdv_opted_in[kMaxDevices];
  KB_CUDA_TRY(opt_in_smem_once(kern_dq, smem_dq, dev, dq_opted_in));
  KB_CUDA_TRY(opt_in_smem_once(kern_dkdv, smem_dkdv, dev, dkdv_opted_in));
  BwdArgs<T> a;
  a.q = make_arg<T>(p.q);
  a.k = make_arg<T>(p.k);
  a.v = make_arg<T>(p.v);
  a.o = make_arg<T>(p.o);
  a.d_o = make_arg<T>(p.d_o);
  a.lse = p.lse;
  a.dq = static_cast<T*>(p.dq);
  a.dk = static_cast<T*>(p.dk);
  a.dv = static_cast<T*>(p.dv);
  a.delta = p.delta_ws;
  a.lens = p.lens;
  a.lens_stride = p.lens_stride;
  a.H = p.H;
  a.T_ = p.T;
  a.c = c;
  a.back = back;
  a.scale_log2 = p.sm_scale * kLog2e;
  a.sm_scale = p.sm_scale;
  dim3 grid_q(kb_cdiv_i32(p.T, BM), p.H, p.B), grid_k(kb_cdiv_i32(p.T, BN), p.H, p.B);
  if (!(p.flags & KB_FLAG_BWD_SKIP_DQ)) {
    kern_dq<<<grid_q, kThreads, smem_dq, s>>>(a);
    KB_LAUNCH_CHECK("sa_bwd_dq_generic_kernel");
  }
  if (!(p.flags & KB_FLAG_BWD_SKIP_DKDV)) {
    kern_dkdv<<<grid_k, kThreads, smem_dkdv, s>>>(a);
    KB_LAUNCH_CHECK("sa_bwd_dkdv_generic_kernel");
  }
  return KB_OK;
}

template <typename T, typename P, typename F>
int dispatch_head_dim(const P& p, F&& f) {
  switch (p.D) {
    case 16: return f(std::integral_constant<int, 16>{});
    case 32: return f(std::integral_constant<int, 32>{});
    case 64: return f(std::integral_constant<int, 64>{});
    case 128: return f(std::integral_constant<int, 128>{});
    case 256: return f(std::integral_constant<int, 256>{});
    default: return KB_ERR_UNSUPPORTED;
  }
}

}  // namespace

int sa_fwd_generic(const kb_sa_fwd_params& p, int32_t c, int32_t back, cudaStream_t s) {
  switch (p.dtype) {
    case KB_F32:
      return dispatch_head_dim<float>(p, [&](auto d) { return launch_fwd<decltype(d)::value, float>(p, c, back, s); });
    case KB_F16:
      return dispatch_head_dim<__half>(p, [&](auto d) { return launch_fwd<decltype(d)::value, __half>(p, c, back, s); });
    case KB_BF16:
      return dispatch_head_dim<__nv_bfloat16>(
          p, [&](auto d) { return launch_fwd<decltype(d)::value, __nv_bfloat16>(p, c, back, s); });
    default:
      return KB_ERR_UNSUPPORTED;
  }
}

int sa_bwd_generic(const kb_sa_bwd_params& p, int32_t c, int32_t back, cudaStream_t s) {
  switch (p.dtype) {
    case KB_F32:
      return dispatch_head_dim<float>(p, [&](auto d) { return launch_bwd<decltype(d)::value, float>(p, c, back, s); });
    case KB_F16:
      return dispatch_head_dim<__half>(p, [&](auto d) { return launch_bwd<decltype(d)::value, __half>(p, c, back, s); });
    case KB_BF16:
      return dispatch_head_dim<__nv_bfloat16>(
          p, [&](auto d) { return launch_bwd<decltype(d)::value, __nv_bfloat16>(p, c, back, s); });
    default:
      return KB_ERR_UNSUPPORTED;
  }
}

}  // namespace kb
