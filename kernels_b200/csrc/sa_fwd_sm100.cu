// Streaming-attention forward for sm_100a: TMA -> shared memory -> tcgen05.mma -> TMEM.
//
// One CTA owns one tile of 128 query rows of one (batch, head) and walks only the live KV
// tiles (64 keys each) of the streaming schedule (schedule.h).  Six warps, three roles:
//   warps 0-3  softmax: thread t owns query row t (= TMEM lane t).  Reads a 128 x 64 block of
//              S from TMEM into registers, keeps the running max / sum, writes P (16-bit) back
//              over S, rescales O when the max moved by more than 2^8, writes O / LSE at the end;
//   warp 4     TMA producer (one lane): Q once, then a ring of K/V tiles;
//   warp 5     MMA issuer (one lane): S = Q K^T (A, B from shared memory), O += P V
//              (A = P from TMEM, B = V from shared memory, MN-major); owns the TMEM allocation.
// S is double buffered in TMEM and the MMA warp issues S(t+1) before P(t) V(t), so the tensor
// pipe works on one KV tile while the softmax warps are busy with the other.
// TMEM columns: [0,64) and [64,128) the two S buffers (fp32; P overlays the first 32 columns of
// each); [128,128+D) O (fp32).  256 columns and ~100 KB of shared memory per CTA keep two CTAs
// resident per SM.
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

constexpr int kBM = 128, kBN = 64;
constexpr int kStages = 2;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColO = 128;
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
  uint8_t k[kStages][kBN * D * 2];
  uint8_t v[kStages][kBN * D * 2];
  uint64_t q_full, k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages], s_ready[2], p_ready[2], pv_done, o_done;
  uint32_t tmem_base;
  int abort_flag;
};

enum WaitSite { kWaitQ = 1, kWaitKEmpty, kWaitVEmpty, kWaitKFull, kWaitVFull, kWaitSReady, kWaitPReady, kWaitPvDone, kWaitEpilogue };

// One 128 x 64 block of scores for the thread's row: online softmax update, P into TMEM.
// kMasked = false is the fast path for blocks in which every element of the warp's rows is live.
template <bool BF16, bool kMasked>
__device__ __forceinline__ void softmax_block(uint32_t t_s, float scale, int k0, int lo, int hi, float& m_used, float& l,
                                              bool& need_rescale, float& alpha) {
  uint32_t s[kBN];
  tmem_ld32(t_s, reinterpret_cast<uint32_t(&)[32]>(s[0]));
  tmem_ld32(t_s + 32, reinterpret_cast<uint32_t(&)[32]>(s[32]));
  tmem_wait_ld();
  if (kMasked) {
#pragma unroll
    for (int i = 0; i < kBN; ++i) {
      const int col = k0 + i;
      s[i] = (col >= lo && col < hi) ? s[i] : 0xff800000u;  // -inf
    }
  }
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int i = 0; i < kBN; i += 4) {
#pragma unroll
    for (int e = 0; e < 4; ++e) mx[e] = fmaxf(mx[e], __uint_as_float(s[i + e]));
  }
  const float m_new = fmaxf(m_used, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale);
  // lazy rescale: keep the old reference maximum unless the new one is > 2^8 larger
  need_rescale = m_new > m_used + kRescaleThreshold;
  alpha = 1.f;
  if (need_rescale) {
    alpha = ex2_approx(m_used - m_new);
    m_used = m_new;
    l *= alpha;
  }
  const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int cc = 0; cc < kBN / 32; ++cc) {
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float p0 = ex2_approx(fmaf(__uint_as_float(s[cc * 32 + 2 * i]), scale, -m_safe));
      const float p1 = ex2_approx(fmaf(__uint_as_float(s[cc * 32 + 2 * i + 1]), scale, -m_safe));
      sum[(2 * i) & 3] += p0;
      sum[(2 * i + 1) & 3] += p1;
      pk[i] = pack16x2<BF16>(p0, p1);
    }
    tmem_st16(t_s + cc * 16, pk);
  }
  l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
}

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
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sm.k_full[s], 1);
      mbar_init(&sm.k_empty[s], 1);
      mbar_init(&sm.v_full[s], 1);
      mbar_init(&sm.v_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.s_ready[i], 1);
      mbar_init(&sm.p_ready[i], kBM);
    }
    mbar_init(&sm.pv_done, 1);
    mbar_init(&sm.o_done, 1);
    sm.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 5) tmem_alloc(&sm.tmem_base, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const WaitCtx ctx{&sm.abort_flag, a.status};
  constexpr uint32_t kQPanelBytes = kBM * 128, kKvPanelBytes = kBN * 128, kKvBytes = kBN * D * 2;
  constexpr int kPanels = D / 64;

  if (warp == 4) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      mbar_expect_tx(&sm.q_full, kBM * D * 2);
#pragma unroll
      for (int p = 0; p < kPanels; ++p) tma_load_4d(sm.q + p * kQPanelBytes, &tm_q, &sm.q_full, p * 64, q0, h, b);
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t % kStages;
        const int k0 = (kr.begin + t) * kBN;
        // K is free again as soon as S(t - kStages) is done, V only after P V: separate rings
        if (t >= kStages && !mbar_wait(&sm.k_empty[s], ((t / kStages) - 1) & 1, ctx, kWaitKEmpty)) break;
        mbar_expect_tx(&sm.k_full[s], kKvBytes);
#pragma unroll
        for (int p = 0; p < kPanels; ++p) tma_load_4d(sm.k[s] + p * kKvPanelBytes, &tm_k, &sm.k_full[s], p * 64, k0, h, b);
        if (t >= kStages && !mbar_wait(&sm.v_empty[s], ((t / kStages) - 1) & 1, ctx, kWaitVEmpty)) break;
        mbar_expect_tx(&sm.v_full[s], kKvBytes);
#pragma unroll
        for (int p = 0; p < kPanels; ++p) tma_load_4d(sm.v[s] + p * kKvPanelBytes, &tm_v, &sm.v_full[s], p * 64, k0, h, b);
      }
    }
  } else if (warp == 5) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(BF16, kBM, kBN, false, false);
      constexpr uint32_t idesc_pv = make_idesc(BF16, kBM, D, false, true);
      const uint32_t q_addr = smem_u32(sm.q);
      bool ok = mbar_wait(&sm.q_full, 0, ctx, kWaitQ);
      for (int t = 0; ok && t <= n_tiles; ++t) {
        if (t < n_tiles) {
          // S(t) = Q K_t^T.  Its TMEM buffer was last read by P(t-2) V(t-2), issued earlier by
          // this thread: MMAs execute in issue order, so no wait is needed for the reuse.
          const int s = t % kStages, buf = t & 1;
          if (!mbar_wait(&sm.k_full[s], (t / kStages) & 1, ctx, kWaitKFull)) break;
          tc_fence_after();
          const uint32_t k_addr = smem_u32(sm.k[s]);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t qo = (kk / 4) * kQPanelBytes + (kk % 4) * 32, ko = (kk / 4) * kKvPanelBytes + (kk % 4) * 32;
            mma_ss(tmem + kColS + buf * kBN, desc_kmajor(q_addr + qo), desc_kmajor(k_addr + ko), idesc_qk, kk > 0);
          }
          mma_commit(&sm.k_empty[s]);
          mma_commit(&sm.s_ready[buf]);
        }
        if (t >= 1) {
          const int u = t - 1, s = u % kStages, buf = u & 1;
          if (!mbar_wait(&sm.p_ready[buf], (u / 2) & 1, ctx, kWaitPReady)) break;
          if (!mbar_wait(&sm.v_full[s], (u / kStages) & 1, ctx, kWaitVFull)) break;
          tc_fence_after();
          const uint32_t v_addr = smem_u32(sm.v[s]);
#pragma unroll
          for (int kk = 0; kk < kBN / 16; ++kk) {
            mma_ts(tmem + kColO, tmem + kColS + buf * kBN + kk * 8, desc_mnmajor(v_addr + kk * 2048, kKvPanelBytes),
                   idesc_pv, u > 0 || kk > 0);
          }
          mma_commit(&sm.v_empty[s]);
          mma_commit(&sm.pv_done);
          if (u == n_tiles - 1) mma_commit(&sm.o_done);
        }
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

    for (int t = 0; t < n_tiles; ++t) {
      const int buf = t & 1;
      const int k0 = (kr.begin + t) * kBN;
      ok = __all_sync(0xffffffffu, mbar_wait(&sm.s_ready[buf], (t / 2) & 1, ctx, kWaitSReady));
      if (!ok) break;
      tc_fence_after();
      const bool warp_full = __all_sync(0xffffffffu, lo <= k0 && k0 + kBN <= hi);
      bool need;
      float alpha;
      if (warp_full)
        softmax_block<BF16, false>(t_lane + kColS + buf * kBN, scale, k0, lo, hi, m_used, l, need, alpha);
      else
        softmax_block<BF16, true>(t_lane + kColS + buf * kBN, scale, k0, lo, hi, m_used, l, need, alpha);
      if (t > 0 && __any_sync(0xffffffffu, need)) {
        // O must not be touched while P(t-1) V(t-1) is still accumulating into it
        ok = __all_sync(0xffffffffu, mbar_wait(&sm.pv_done, (t - 1) & 1, ctx, kWaitPvDone));
        if (!ok) break;
        tc_fence_after();
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
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&sm.p_ready[buf]);
    }

    // A parity wait on pv_done could be two phases behind here (only P(n-3) V(n-3) is known to be
    // complete), which a parity bit cannot tell apart: the last accumulation has its own barrier.
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&sm.o_done, 0, ctx, kWaitEpilogue));
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
