// Streaming-attention forward for sm_100a: TMA -> shared memory -> tcgen05.mma -> TMEM.
//
// One CTA owns one tile of 128 query rows of one (batch, head) and walks only the live KV
// tiles of the streaming schedule (schedule.h).  Six warps, three roles:
//   warps 0-3  softmax: thread t owns query row t (= TMEM lane t).  Reads S from TMEM, keeps the
//              running max / sum, writes P (16-bit) back over S, rescales O when the max
//              moved by more than 2^8, and writes O / LSE at the end;
//   warp 4     TMA producer (one lane): Q once, then K and V tiles;
//   warp 5     MMA issuer (one lane): S = Q K^T (A, B from shared memory), O += P V
//              (A = P from TMEM, B = V from shared memory, MN-major); owns the TMEM allocation.
// TMEM columns: [0,128) S (fp32), overlaid by P in [0,64); [128,128+D) O (fp32).  256 columns
// per CTA and one K and one V buffer keep two CTAs resident per SM: while one CTA is in its
// softmax the other one's MMAs use the tensor pipe.
//
// Masking uses the fact that the live keys of a query row form one interval
// [max(0, i/c - back) * c, min((i/c + 1) * c, len)), which is the element form of the mask
// (i < len, j < len, 0 <= i/c - j/c <= back).
//
// Reference semantics: src/streaming_attention/kernel.py:205-430 (online softmax in base 2,
// P cast to the input type before P V, LSE = m + log2(l)).
#include <math.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "sm100_host.h"

namespace kb {
namespace {

using namespace sm100;

constexpr int kBM = 128, kBN = 128;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColP = 0, kColO = 128;
constexpr float kRescaleThreshold = 8.f;  // log2 units

struct FwdArgs {
  void* o;
  float* lse;
  const int32_t* lens;
  int64_t lens_stride;
  int32_t H, T, c, back;
  float scale_log2;
  int32_t* status;
};

template <int D>
struct alignas(1024) FwdSmem {
  uint8_t q[kBM * D * 2];
  uint8_t k[kBN * D * 2];
  uint8_t v[kBN * D * 2];
  uint64_t q_full, k_full, v_full, k_empty, v_empty, s_ready, p_ready, pv_done;
  uint32_t tmem_base;
  int abort_flag;
};

enum WaitSite { kWaitQ = 1, kWaitKEmpty, kWaitVEmpty, kWaitKFull, kWaitVFull, kWaitSReady, kWaitPReady, kWaitPvDone, kWaitEpilogue };

template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads, 2)
sa_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const FwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  FwdSmem<D>& sm = *reinterpret_cast<FwdSmem<D>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * kBM;
  const int T = a.T;
  const int len = a.lens ? kb_clamp_len(a.lens[(int64_t)b * a.lens_stride], T) : T;
  const int64_t bh = (int64_t)b * a.H + h;
  uint16_t* o_slice = static_cast<uint16_t*>(a.o) + bh * T * D;
  float* lse_slice = a.lse ? a.lse + bh * T : nullptr;

  const KbTileRange kr = kb_fwd_kv_range(q0, kBM, kBN, len, a.c, a.back);
  if (kr.begin >= kr.end) {
    // the whole q tile lies in the padding: its rows are zeros
    if (threadIdx.x < kBM && q0 + (int)threadIdx.x < T) {
      uint4* row = reinterpret_cast<uint4*>(o_slice + (int64_t)(q0 + threadIdx.x) * D);
#pragma unroll
      for (int i = 0; i < D * 2 / 16; ++i) row[i] = make_uint4(0, 0, 0, 0);
      if (lse_slice) lse_slice[q0 + threadIdx.x] = 0.f;
    }
    return;
  }
  const int n_tiles = kr.end - kr.begin;

  if (threadIdx.x == 0) {
    mbar_init(&sm.q_full, 1);
    mbar_init(&sm.k_full, 1);
    mbar_init(&sm.v_full, 1);
    mbar_init(&sm.k_empty, 1);
    mbar_init(&sm.v_empty, 1);
    mbar_init(&sm.s_ready, 1);
    mbar_init(&sm.p_ready, kBM);
    mbar_init(&sm.pv_done, 1);
    sm.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 5) tmem_alloc(&sm.tmem_base, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const WaitCtx ctx{&sm.abort_flag, a.status};
  constexpr uint32_t kTileBytes = kBN * D * 2, kPanelBytes = kBN * 128;
  constexpr int kPanels = D / 64;

  if (warp == 4) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      mbar_expect_tx(&sm.q_full, kBM * D * 2);
#pragma unroll
      for (int p = 0; p < kPanels; ++p) tma_load_4d(sm.q + p * kPanelBytes, &tm_q, &sm.q_full, p * 64, q0, h, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int k0 = (kr.begin + j) * kBN;
        if (j > 0 && !mbar_wait(&sm.k_empty, (j - 1) & 1, ctx, kWaitKEmpty)) break;
        mbar_expect_tx(&sm.k_full, kTileBytes);
#pragma unroll
        for (int p = 0; p < kPanels; ++p) tma_load_4d(sm.k + p * kPanelBytes, &tm_k, &sm.k_full, p * 64, k0, h, b);
        if (j > 0 && !mbar_wait(&sm.v_empty, (j - 1) & 1, ctx, kWaitVEmpty)) break;
        mbar_expect_tx(&sm.v_full, kTileBytes);
#pragma unroll
        for (int p = 0; p < kPanels; ++p) tma_load_4d(sm.v + p * kPanelBytes, &tm_v, &sm.v_full, p * 64, k0, h, b);
      }
    }
  } else if (warp == 5) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(BF16, kBM, kBN, false, false);
      constexpr uint32_t idesc_pv = make_idesc(BF16, kBM, D, false, true);
      const uint32_t q_addr = smem_u32(sm.q), k_addr = smem_u32(sm.k), v_addr = smem_u32(sm.v);
      bool ok = mbar_wait(&sm.q_full, 0, ctx, kWaitQ);
      for (int j = 0; ok && j < n_tiles; ++j) {
        // S/P columns are reused: the previous P V must have drained them
        if (j > 0 && !mbar_wait(&sm.pv_done, (j - 1) & 1, ctx, kWaitPvDone)) break;
        if (!mbar_wait(&sm.k_full, j & 1, ctx, kWaitKFull)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * kPanelBytes + (kk % 4) * 32;
          mma_ss(tmem + kColS, desc_kmajor(q_addr + off), desc_kmajor(k_addr + off), idesc_qk, kk > 0);
        }
        mma_commit(&sm.k_empty);
        mma_commit(&sm.s_ready);
        if (!mbar_wait(&sm.p_ready, j & 1, ctx, kWaitPReady)) break;
        if (!mbar_wait(&sm.v_full, j & 1, ctx, kWaitVFull)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk) {
          mma_ts(tmem + kColO, tmem + kColP + kk * 8, desc_mnmajor(v_addr + kk * 16 * 128, kPanelBytes), idesc_pv,
                 j > 0 || kk > 0);
        }
        mma_commit(&sm.v_empty);
        mma_commit(&sm.pv_done);
      }
    }
  } else {
    // ------------------------------ softmax + epilogue ------------------------------
    const int row = threadIdx.x;
    const int qi = q0 + row;
    int lo = 0, hi = 0;
    if (qi < len) {
      const int qc = qi / a.c;
      lo = kb_max_i32(0, qc - a.back) * a.c;
      const int64_t h64 = (int64_t)(qc + 1) * a.c;
      hi = h64 < len ? (int)h64 : len;
    }
    const uint32_t t_lane = tmem + ((uint32_t)(warp * 32) << 16);
    const float scale = a.scale_log2;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;

    for (int j = 0; j < n_tiles; ++j) {
      const int k0 = (kr.begin + j) * kBN;
      ok = __all_sync(0xffffffffu, mbar_wait(&sm.s_ready, j & 1, ctx, kWaitSReady));
      if (!ok) break;
      tc_fence_after();
      const bool warp_full = __all_sync(0xffffffffu, lo <= k0 && k0 + kBN <= hi);

      // pass 1: row maximum of the raw scores
      float mx = -INFINITY;
#pragma unroll
      for (int cc = 0; cc < kBN / 32; ++cc) {
        uint32_t r[32];
        tmem_ld32(t_lane + kColS + cc * 32, r);
        tmem_wait_ld();
        if (warp_full) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = k0 + cc * 32 + i;
            mx = fmaxf(mx, (col >= lo && col < hi) ? __uint_as_float(r[i]) : -INFINITY);
          }
        }
      }
      const float m_new = fmaxf(m_used, mx * scale);
      // lazy rescale: keep the old reference maximum unless the new one is > 2^8 larger
      const bool need = m_new > m_used + kRescaleThreshold;
      float alpha = 1.f;
      if (need) {
        alpha = ex2_approx(m_used - m_new);
        m_used = m_new;
        l *= alpha;
      }
      if (j > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t r[32];
          tmem_ld32(t_lane + kColO + cc * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(t_lane + kColO + cc * 32, r);
        }
      }
      const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;

      // pass 2: P = 2^(S * scale - m), row sum, 16-bit P back into TMEM over S
#pragma unroll
      for (int cc = 0; cc < kBN / 32; ++cc) {
        uint32_t r[32];
        tmem_ld32(t_lane + kColS + cc * 32, r);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = ex2_approx(fmaf(__uint_as_float(r[2 * i]), scale, -m_safe));
          float p1 = ex2_approx(fmaf(__uint_as_float(r[2 * i + 1]), scale, -m_safe));
          if (!warp_full) {
            const int col = k0 + cc * 32 + 2 * i;
            p0 = (col >= lo && col < hi) ? p0 : 0.f;
            p1 = (col + 1 >= lo && col + 1 < hi) ? p1 : 0.f;
          }
          l += p0 + p1;
          pk[i] = pack16x2<BF16>(p0, p1);
        }
        tmem_st16(t_lane + kColP + cc * 16, pk);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&sm.p_ready);
    }

    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&sm.pv_done, (n_tiles - 1) & 1, ctx, kWaitEpilogue));
    if (ok) {
      tc_fence_after();
      const bool valid = qi < len;
      const float inv = valid ? 1.f / l : 0.f;
#pragma unroll
      for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t r[32];
        tmem_ld32(t_lane + kColO + cc * 32, r);
        tmem_wait_ld();
        if (qi < T) {
          uint4* dst = reinterpret_cast<uint4*>(o_slice + (int64_t)qi * D + cc * 32);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack16x2<BF16>(__uint_as_float(r[8 * g + 0]) * inv, __uint_as_float(r[8 * g + 1]) * inv);
            w.y = pack16x2<BF16>(__uint_as_float(r[8 * g + 2]) * inv, __uint_as_float(r[8 * g + 3]) * inv);
            w.z = pack16x2<BF16>(__uint_as_float(r[8 * g + 4]) * inv, __uint_as_float(r[8 * g + 5]) * inv);
            w.w = pack16x2<BF16>(__uint_as_float(r[8 * g + 6]) * inv, __uint_as_float(r[8 * g + 7]) * inv);
            dst[g] = w;
          }
        }
      }
      if (lse_slice && qi < T) lse_slice[qi] = valid ? m_used + log2f(l) : 0.f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    if (sm.abort_flag) __nanosleep(1000000);  // let copies still in flight land before the CTA goes away
    tmem_dealloc(tmem, kTmemCols);
  }
}

template <int D, bool BF16>
int launch(const kb_sa_fwd_params& p, int32_t c, int32_t back, cudaStream_t s) {
  CUtensorMap tm_q, tm_k, tm_v;
  if (!make_tile_map_4d(&tm_q, p.q, p.B, p.H, p.T, D, kBM) || !make_tile_map_4d(&tm_k, p.k, p.B, p.H, p.T, D, kBN) ||
      !make_tile_map_4d(&tm_v, p.v, p.B, p.H, p.T, D, kBN))
    return KB_ERR_UNSUPPORTED;
  auto kern = sa_fwd_sm100_kernel<D, BF16>;
  constexpr size_t smem = sizeof(FwdSmem<D>) + 1024;
  KB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  FwdArgs a;
  a.o = p.o;
  a.lse = p.lse;
  a.lens = p.lens;
  a.lens_stride = p.lens_stride;
  a.H = p.H;
  a.T = p.T;
  a.c = c;
  a.back = back;
  a.scale_log2 = p.sm_scale * kLog2e;
  a.status = p.status;
  dim3 grid(kb_cdiv_i32(p.T, kBM), p.H, p.B);
  kern<<<grid, kThreads, smem, s>>>(tm_q, tm_k, tm_v, a);
  KB_LAUNCH_CHECK("sa_fwd_sm100_kernel");
  return KB_OK;
}

}  // namespace

int sa_fwd_sm100(const kb_sa_fwd_params& p, int32_t c, int32_t back, cudaStream_t s) {
  if (!(p.sm_scale > 0.f) || reinterpret_cast<uintptr_t>(p.o) % 16) return KB_ERR_UNSUPPORTED;
  const bool bf16 = p.dtype == KB_BF16;
  if (p.D == 64) return bf16 ? launch<64, true>(p, c, back, s) : launch<64, false>(p, c, back, s);
  if (p.D == 128) return bf16 ? launch<128, true>(p, c, back, s) : launch<128, false>(p, c, back, s);
  return KB_ERR_UNSUPPORTED;
}

}  // namespace kb
