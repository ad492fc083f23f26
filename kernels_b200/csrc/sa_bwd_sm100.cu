// Streaming-attention backward for sm_100a: one kernel template, two passes.
//
//   dQ pass    (kDQ = true):  a CTA keeps 128 query rows (Q, dO) in shared memory and streams
//                             128-row K/V tiles over the forward schedule.  It also produces
//                             delta = rowsum(O * dO) for its rows and leaves it in the
//                             workspace for the other pass.
//   dK/dV pass (kDQ = false): a CTA keeps 128 key rows (K, V) and streams 128-row Q/dO tiles
//                             over the transposed schedule.
// Both passes have the same shape.  With X the stationary operands (A1, A2) and Y_t the
// streamed ones (B1, B2):
//   S  = A1 * B1^T   (scores, 128 x 128)         dP = A2 * B2^T   (128 x 128)
//   P  = 2^(S * scale - lse[q])                  dS = P * (dP - delta[q])      (masked -> 0)
//   dQ pass:    dQ += dS * K_t                   dK/dV pass: dV += P * dO_t,  dK += dS * Q_t
// S and dP live in TMEM; P and dS are written back over them as 16-bit values and feed the
// accumulating MMAs as the A operand straight from TMEM; the streamed tile in shared memory is
// read K-major by the first two MMAs and MN-major by the accumulating ones.
//
// The tensor pipe and the compute warps overlap by splitting each tile into two phases:
//   dK/dV pass MMA order:  S(0) dP(0) | dV(t) S(t+1) dK(t) dP(t+1) | ...
//       while the compute warps turn S(t+1) into P(t+1) the pipe runs dK(t), dP(t+1);
//       while they turn dP(t+1) into dS(t+1) it runs dV(t+1), S(t+2).
//   dQ pass MMA order:     S(0) dP(0) S(1) | dQ(t) dP(t+1) S(t+2) | ...   (S double buffered)
// MMAs execute in issue order, so a buffer that a later MMA overwrites needs no wait on the
// earlier MMA that reads it; waits exist only where the compute warps or TMA are involved.
//
// Roles: warps 0-7 compute (two warpgroups; a thread owns row (warp % 4) * 32 + lane = its TMEM
// lane, and warpgroup g the columns [64 g, 64 g + 64) of every tile), warp 8 TMA producer (plus
// the per-column lse/delta staging of the dK/dV pass), warp 9 MMA issuer and TMEM owner.
// TMEM columns: S at 0 (second S buffer of the dQ pass at 384), dP at 128, accumulator 1 at
// 256, accumulator 2 (dK) at 384.
//
// Reference semantics: src/streaming_attention/kernel.py:453-514 (delta), 639-773 and
// 941-1023 (dQ), 777-937 and 1027-1129 (dK/dV).  No atomics: results are bitwise repeatable.
#include <math.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "sm100_host.h"
#include "tiles.h"

namespace kb {
#ifdef KB_TRACE
// Debug build only (-DKB_TRACE): clock64 stamps of one CTA's pipeline events, read back by
// kb_debug_trace().  [role: 0 producer, 1 MMA, 2 compute warp 0][tile][slot]
__device__ long long g_trace[3][64][8];
#define KB_TR(role, t, slot)                                      \
  do {                                                            \
    if (trace_cta && (t) < 64) g_trace[role][t][slot] = clock64(); \
  } while (0)
#else
#define KB_TR(role, t, slot) \
  do {                       \
  } while (0)
#endif
namespace {

using namespace sm100;

constexpr int kBX = tiles::kTwoPassStationary;  // stationary rows per CTA
constexpr int kBY = tiles::kTwoPassStreamed;    // streamed rows per tile
constexpr int kStagesB1 = tiles::kTwoPassStagesFirst, kStagesB2 = tiles::kTwoPassStagesSecond;
static_assert(kBX == 128 && kBY == 128, "the TMEM column map assumes 128 x 128 score blocks");
constexpr int kComputeWarps = 8;
constexpr int kComputeThreads = kComputeWarps * 32;
constexpr int kThreads = (kComputeWarps + 2) * 32;
constexpr int kProducerWarp = kComputeWarps, kMmaWarp = kComputeWarps + 1;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColS1 = 384, kColDP = 128, kColAcc1 = 256, kColAcc2 = 384;

struct BwdArgs {
  // dQ pass: o / d_o rows for delta (element strides of b, h, t; unit inner stride)
  const uint16_t* o;
  const uint16_t* d_o;
  int64_t o_sb, o_sh, o_st, do_sb, do_sh, do_st;
  const float* lse;
  float* delta;
  void* out1;  // dQ pass: dq.  dK/dV pass: dv
  void* out2;  // dK/dV pass: dk
  const int32_t* lens;
  int64_t lens_stride;
  int32_t H, T, c, back;
  float scale_log2, sm_scale;
  int32_t* status;
};

// Shared memory of one CTA.  At D = 128 this is exactly the 227 KB a CTA may have, which is why
// the base of dynamic shared memory itself must be 1024-byte aligned (checked at run time)
// instead of being rounded up inside a larger allocation.
template <int D>
struct alignas(1024) BwdSmem {
  uint8_t a1[kBX * D * 2];
  uint8_t a2[kBX * D * 2];
  uint8_t b1[kStagesB1][kBY * D * 2];
  uint8_t b2[kStagesB2][kBY * D * 2];
  alignas(16) float lse_s[2][kBY];
  alignas(16) float delta_s[2][kBY];
  uint64_t x_full, b1_full[kStagesB1], b1_empty[kStagesB1], b2_full[kStagesB2], b2_empty[kStagesB2];
  uint64_t s_ready[2], dp_ready, p_ready, ds_ready[2], stats_full[2], acc_done, staged;
  uint32_t tmem_base;
  int abort_flag;
};

enum WaitSite { kWX = 21, kWB1Empty, kWB2Empty, kWStats, kWStatsFull, kWB1Full, kWB2Full, kWSReady, kWDpReady, kWPReady, kWDsReady, kWAccDone, kWStaged };
constexpr int kErrSmemAlign = 41;

template <int D, bool BF16, bool kDQ>
__global__ void __launch_bounds__(kThreads, 1)
sa_bwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_a1, const __grid_constant__ CUtensorMap tm_a2,
                    const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_b2,
                    const __grid_constant__ CUtensorMap tm_out1, const __grid_constant__ CUtensorMap tm_out2,
                    const BwdArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  BwdSmem<D>& sm = *reinterpret_cast<BwdSmem<D>*>(smem_raw);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y, x0 = blockIdx.x * kBX;
  const int T = a.T;
  const int len = a.lens ? kb_clamp_len(a.lens[(int64_t)b * a.lens_stride], T) : T;
  const int64_t bh = (int64_t)b * a.H + h;
  uint16_t* out1 = static_cast<uint16_t*>(a.out1) + bh * T * D;
  uint16_t* out2 = kDQ ? nullptr : static_cast<uint16_t*>(a.out2) + bh * T * D;

  if (smem_u32(smem_raw) & 1023u) {
    // swizzled operand tiles need a 1024-byte aligned base: report instead of computing garbage
    if (threadIdx.x == 0 && a.status) {
      atomicExch(a.status, KB_ERR_DEVICE_TIMEOUT);
      atomicExch(a.status + 1, kErrSmemAlign);
    }
    return;
  }

  // streamed tiles [begin, end) in units of kBY rows
  const KbTileRange yr = kDQ ? kb_fwd_kv_range(x0, kBX, kBY, len, a.c, a.back) : kb_bwd_q_range(x0, kBY, kBX, len, a.c, a.back);
  if (yr.begin >= yr.end) {
    // the whole stationary tile lies in the padding: its gradients are zeros
    if (threadIdx.x < kBX && x0 + (int)threadIdx.x < T) {
      const int64_t r = x0 + threadIdx.x;
      uint4* row1 = reinterpret_cast<uint4*>(out1 + r * D);
#pragma unroll
      for (int i = 0; i < D * 2 / 16; ++i) row1[i] = make_uint4(0, 0, 0, 0);
      if (kDQ) {
        a.delta[bh * T + r] = 0.f;
      } else {
        uint4* row2 = reinterpret_cast<uint4*>(out2 + r * D);
#pragma unroll
        for (int i = 0; i < D * 2 / 16; ++i) row2[i] = make_uint4(0, 0, 0, 0);
      }
    }
    return;
  }
  const int n_tiles = yr.end - yr.begin;
#ifdef KB_TRACE
  const bool trace_cta = blockIdx.x == 60 && blockIdx.y == 0 && blockIdx.z == 0 && (kDQ == (KB_TRACE != 0));
#endif

  if (threadIdx.x == 0) {
    mbar_init(&sm.x_full, 1);
    for (int s = 0; s < kStagesB1; ++s) {
      mbar_init(&sm.b1_full[s], 1);
      mbar_init(&sm.b1_empty[s], 1);
    }
    for (int s = 0; s < kStagesB2; ++s) {
      mbar_init(&sm.b2_full[s], 1);
      mbar_init(&sm.b2_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.s_ready[i], 1);
      mbar_init(&sm.ds_ready[i], kComputeThreads);
      mbar_init(&sm.stats_full[i], kDQ ? kComputeThreads : 32);
    }
    mbar_init(&sm.dp_ready, 1);
    mbar_init(&sm.p_ready, kComputeThreads);
    mbar_init(&sm.acc_done, 1);
    mbar_init(&sm.staged, kComputeThreads);
    sm.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kMmaWarp) tmem_alloc(&sm.tmem_base, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const WaitCtx ctx{&sm.abort_flag, a.status};
  constexpr int kPanels = D / 64;
  constexpr uint32_t kPanelBytes = 128 * 128;  // 128 rows x 128 bytes, both operand kinds
  constexpr uint32_t kTileBytes = 128 * D * 2;

  if (warp == kProducerWarp) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&tm_a1);
      prefetch_tensormap(&tm_a2);
      prefetch_tensormap(&tm_b1);
      prefetch_tensormap(&tm_b2);
      mbar_expect_tx(&sm.x_full, 2 * kTileBytes);
#pragma unroll
      for (int p = 0; p < kPanels; ++p) {
        tma_load_4d(sm.a1 + p * kPanelBytes, &tm_a1, &sm.x_full, p * 64, x0, h, b);
        tma_load_4d(sm.a2 + p * kPanelBytes, &tm_a2, &sm.x_full, p * 64, x0, h, b);
      }
    }
    for (int t = 0; t < n_tiles; ++t) {
      const int s1 = t % kStagesB1, s2 = t % kStagesB2;
      const int y0 = (yr.begin + t) * kBY;
      bool ok = true;
      if (lane == 0) {
        KB_TR(0, t, 0);
        if (t >= kStagesB1) ok = mbar_wait(&sm.b1_empty[s1], ((t / kStagesB1) - 1) & 1, ctx, kWB1Empty);
        if (ok) {
          mbar_expect_tx(&sm.b1_full[s1], kTileBytes);
#pragma unroll
          for (int p = 0; p < kPanels; ++p) tma_load_4d(sm.b1[s1] + p * kPanelBytes, &tm_b1, &sm.b1_full[s1], p * 64, y0, h, b);
          KB_TR(0, t, 1);
          if (t >= kStagesB2) ok = mbar_wait(&sm.b2_empty[s2], ((t / kStagesB2) - 1) & 1, ctx, kWB2Empty);
          KB_TR(0, t, 2);
        }
        if (ok) {
          mbar_expect_tx(&sm.b2_full[s2], kTileBytes);
#pragma unroll
          for (int p = 0; p < kPanels; ++p) tma_load_4d(sm.b2[s2] + p * kPanelBytes, &tm_b2, &sm.b2_full[s2], p * 64, y0, h, b);
        }
      }
      if (!kDQ) {
        // per-column statistics (lse, delta) of the streamed query rows, two slots deep: slot t & 1
        // was last read while dS(t-2) was formed
        if (ok && t >= 2) ok = mbar_wait(&sm.ds_ready[t & 1], ((t / 2) - 1) & 1, ctx, kWStats);
        if (!__all_sync(0xffffffffu, ok)) break;
#pragma unroll
        for (int i = 0; i < kBY / 32; ++i) {
          const int r = y0 + lane + 32 * i;
          const bool valid = r < len;
          sm.lse_s[t & 1][lane + 32 * i] = valid ? a.lse[bh * T + r] : 0.f;
          sm.delta_s[t & 1][lane + 32 * i] = valid ? a.delta[bh * T + r] : 0.f;
        }
        mbar_arrive(&sm.stats_full[t & 1]);
      } else if (!__all_sync(0xffffffffu, ok)) {
        break;
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_z = make_idesc(BF16, kBX, kBY, false, false);
      constexpr uint32_t idesc_acc = make_idesc(BF16, kBX, D, false, true);
      const uint32_t a1_addr = smem_u32(sm.a1), a2_addr = smem_u32(sm.a2);

      // S(t) = A1 * B1_t^T into S buffer `sbuf`
      auto issue_s = [&](int t, int sbuf) -> bool {
        const int s1 = t % kStagesB1;
        KB_TR(1, t, 0);
        if (!mbar_wait(&sm.b1_full[s1], (t / kStagesB1) & 1, ctx, kWB1Full)) return false;
        KB_TR(1, t, 1);
        tc_fence_after();
        const uint32_t b_addr = smem_u32(sm.b1[s1]);
        const uint32_t d_col = tmem + (sbuf ? kColS1 : kColS);
        uint32_t a_lo = desc_lo_kmajor(a1_addr), b_lo = desc_lo_kmajor(b_addr);
#pragma unroll 1
        for (int h = 0; h < D / 64; ++h, a_lo += kPanelBytes >> 4, b_lo += kPanelBytes >> 4) {
#pragma unroll
          for (int i = 0; i < 4; ++i) mma_ss_lo(d_col, a_lo + 2 * i, b_lo + 2 * i, idesc_z, h > 0 || i > 0);
        }
        mma_commit(&sm.s_ready[sbuf]);
        KB_TR(1, t, 2);
        return true;
      };
      // dP(t) = A2 * B2_t^T
      auto issue_dp = [&](int t) -> bool {
        const int s2 = t % kStagesB2;
        if (!mbar_wait(&sm.b2_full[s2], (t / kStagesB2) & 1, ctx, kWB2Full)) return false;
        KB_TR(1, t, 3);
        tc_fence_after();
        const uint32_t b_addr = smem_u32(sm.b2[s2]);
        uint32_t a_lo = desc_lo_kmajor(a2_addr), b_lo = desc_lo_kmajor(b_addr);
#pragma unroll 1
        for (int h = 0; h < D / 64; ++h, a_lo += kPanelBytes >> 4, b_lo += kPanelBytes >> 4) {
#pragma unroll
          for (int i = 0; i < 4; ++i) mma_ss_lo(tmem + kColDP, a_lo + 2 * i, b_lo + 2 * i, idesc_z, h > 0 || i > 0);
        }
        if (kDQ) mma_commit(&sm.b2_empty[s2]);  // V_t has no other reader in the dQ pass
        mma_commit(&sm.dp_ready);
        KB_TR(1, t, 4);
        return true;
      };
      // acc += A(tmem, 16-bit at `a_col`) * B(smem tile at b_addr, MN-major)
      auto issue_acc = [&](uint32_t acc_col, uint32_t a_col, uint32_t b_addr, bool first_tile) {
        // 16 reduction rows = 8 packed columns; rows [64 g, 64 g + 64) sit at columns 64 g ..
        uint32_t a = tmem + a_col, b_lo = desc_lo_mnmajor(b_addr, kPanelBytes);
#pragma unroll 1
        for (int h = 0; h < kBY / 64; ++h, a += 64, b_lo += 4 * (2048 >> 4)) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            mma_ts_lo(tmem + acc_col, a + 8 * i, b_lo + i * (2048 >> 4), idesc_acc, !first_tile || h > 0 || i > 0);
        }
      };

      bool ok = mbar_wait(&sm.x_full, 0, ctx, kWX);
      if (kDQ) {
        ok = ok && issue_s(0, 0) && issue_dp(0);
        if (ok && n_tiles > 1) ok = issue_s(1, 1);
        for (int t = 0; ok && t < n_tiles; ++t) {
          const int s1 = t % kStagesB1;
          KB_TR(1, t, 5);
          if (!mbar_wait(&sm.ds_ready[t & 1], (t / 2) & 1, ctx, kWDsReady)) break;
          KB_TR(1, t, 6);
          tc_fence_after();
          issue_acc(kColAcc1, kColDP, smem_u32(sm.b1[s1]), t == 0);  // dQ += dS * K_t
          mma_commit(&sm.b1_empty[s1]);
          KB_TR(1, t, 7);
          if (t == n_tiles - 1) mma_commit(&sm.acc_done);
          if (t + 1 < n_tiles && !issue_dp(t + 1)) break;
          if (t + 2 < n_tiles && !issue_s(t + 2, t & 1)) break;
        }
      } else {
        ok = ok && issue_s(0, 0) && issue_dp(0);
        for (int t = 0; ok && t < n_tiles; ++t) {
          const int s1 = t % kStagesB1, s2 = t % kStagesB2;
          if (!mbar_wait(&sm.p_ready, t & 1, ctx, kWPReady)) break;
          tc_fence_after();
          issue_acc(kColAcc1, kColS, smem_u32(sm.b2[s2]), t == 0);  // dV += P * dO_t
          mma_commit(&sm.b2_empty[s2]);
          if (t + 1 < n_tiles && !issue_s(t + 1, 0)) break;
          KB_TR(1, t, 5);
          if (!mbar_wait(&sm.ds_ready[t & 1], (t / 2) & 1, ctx, kWDsReady)) break;
          KB_TR(1, t, 6);
          tc_fence_after();
          issue_acc(kColAcc2, kColDP, smem_u32(sm.b1[s1]), t == 0);  // dK += dS * Q_t
          mma_commit(&sm.b1_empty[s1]);
          KB_TR(1, t, 7);
          if (t == n_tiles - 1) mma_commit(&sm.acc_done);
          if (t + 1 < n_tiles && !issue_dp(t + 1)) break;
        }
      }
    }
  } else {
    // ------------------------------ compute warps + epilogue ------------------------------
    const int row = (warp & 3) * 32 + lane;
    const int half = warp >> 2;  // which 64 columns of each tile this warpgroup owns
    const int xi = x0 + row;
    // live columns of this row form one interval [lo, hi)
    int lo = 0, hi = 0;
    if (xi < len) {
      const int xc = xi / a.c;
      if (kDQ) {
        lo = kb_max_i32(0, xc - a.back) * a.c;
        const int64_t h64 = (int64_t)(xc + 1) * a.c;
        hi = h64 < len ? (int)h64 : len;
      } else {
        lo = xc * a.c;
        const int64_t h64 = (int64_t)(xc + a.back + 1) * a.c;
        hi = h64 < len ? (int)h64 : len;
      }
    }
    const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const float scale = a.scale_log2;

    float lse_r = 0.f, delta_r = 0.f;
    bool ok = true;
    if (kDQ) {
      // delta = rowsum(O * dO) for the 128 rows of the tile, read cooperatively: a group of D/8
      // lanes reads one row as 16-byte chunks (fully coalesced), warp w covers rows 16 w .. 16 w + 15,
      // and the row sums travel to their owner threads through shared memory.
      constexpr int kLanesPerRow = D / 8, kRowsPerIter = 32 / kLanesPerRow, kIters = 16 / kRowsPerIter;
      const int sub = lane / kLanesPerRow, chunk = lane % kLanesPerRow;
      const uint16_t* o_base = a.o + b * a.o_sb + h * a.o_sh;
      const uint16_t* g_base = a.d_o + b * a.do_sb + h * a.do_sh;
      uint4 ov[kIters], gv[kIters];
#pragma unroll
      for (int it = 0; it < kIters; ++it) {
        const int r = x0 + 16 * warp + it * kRowsPerIter + sub;
        ov[it] = gv[it] = make_uint4(0, 0, 0, 0);
        if (r < len) {
          ov[it] = __ldg(reinterpret_cast<const uint4*>(o_base + (int64_t)r * a.o_st) + chunk);
          gv[it] = __ldg(reinterpret_cast<const uint4*>(g_base + (int64_t)r * a.do_st) + chunk);
        }
      }
#pragma unroll
      for (int it = 0; it < kIters; ++it) {
        const uint32_t ow[4] = {ov[it].x, ov[it].y, ov[it].z, ov[it].w}, gw[4] = {gv[it].x, gv[it].y, gv[it].z, gv[it].w};
        float part = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          float o0, o1, g0, g1;
          if (BF16) {
            o0 = __uint_as_float(ow[w] << 16);
            o1 = __uint_as_float(ow[w] & 0xffff0000u);
            g0 = __uint_as_float(gw[w] << 16);
            g1 = __uint_as_float(gw[w] & 0xffff0000u);
          } else {
            const __half2 oh = *reinterpret_cast<const __half2*>(&ow[w]), gh = *reinterpret_cast<const __half2*>(&gw[w]);
            o0 = __low2float(oh);
            o1 = __high2float(oh);
            g0 = __low2float(gh);
            g1 = __high2float(gh);
          }
          part = fmaf(o0, g0, part);
          part = fmaf(o1, g1, part);
        }
#pragma unroll
        for (int off = kLanesPerRow / 2; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
        if (chunk == 0) {
          const int rr = 16 * warp + it * kRowsPerIter + sub;
          sm.delta_s[0][rr] = part;
          if (x0 + rr < T) a.delta[bh * T + x0 + rr] = part;
        }
      }
      mbar_arrive(&sm.stats_full[0]);
      if (xi < len) lse_r = a.lse[bh * T + xi];
      ok = __all_sync(0xffffffffu, mbar_wait(&sm.stats_full[0], 0, ctx, kWStatsFull));
      delta_r = sm.delta_s[0][row];
    }

    for (int t = 0; ok && t < n_tiles; ++t) {
      const int y0 = (yr.begin + t) * kBY + half * 64;  // first column this thread handles
      const int sbuf = kDQ ? (t & 1) : 0;
      const uint32_t t_s = t_lane + (sbuf ? kColS1 : kColS) + half * 64;
      const uint32_t t_dp = t_lane + kColDP + half * 64;
      const float* lse_c = sm.lse_s[t & 1] + half * 64;
      const float* delta_c = sm.delta_s[t & 1] + half * 64;

      // ---- phase 1: P = 2^(S * scale - lse) for this thread's 64 columns
      if (threadIdx.x == 0) KB_TR(2, t, 0);
      ok = __all_sync(0xffffffffu, mbar_wait(&sm.s_ready[sbuf], kDQ ? (t / 2) & 1 : t & 1, ctx, kWSReady));
      if (ok && !kDQ) ok = __all_sync(0xffffffffu, mbar_wait(&sm.stats_full[t & 1], (t / 2) & 1, ctx, kWStatsFull));
      if (!ok) break;
      tc_fence_after();
      if (threadIdx.x == 0) KB_TR(2, t, 1);
      const bool warp_full = __all_sync(0xffffffffu, lo <= y0 && y0 + 64 <= hi);
      float p[64];
      {
        uint32_t s[64];
        tmem_ld32(t_s, reinterpret_cast<uint32_t(&)[32]>(s[0]));
        tmem_ld32(t_s + 32, reinterpret_cast<uint32_t(&)[32]>(s[32]));
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
          float4 lv = make_float4(lse_r, lse_r, lse_r, lse_r);
          if (!kDQ) lv = *reinterpret_cast<const float4*>(lse_c + i);
          p[i + 0] = ex2_approx(fmaf(__uint_as_float(s[i + 0]), scale, -lv.x));
          p[i + 1] = ex2_approx(fmaf(__uint_as_float(s[i + 1]), scale, -lv.y));
          p[i + 2] = ex2_approx(fmaf(__uint_as_float(s[i + 2]), scale, -lv.z));
          p[i + 3] = ex2_approx(fmaf(__uint_as_float(s[i + 3]), scale, -lv.w));
        }
        if (!warp_full) {
#pragma unroll
          for (int i = 0; i < 64; ++i) p[i] = (y0 + i >= lo && y0 + i < hi) ? p[i] : 0.f;
        }
      }
      if (!kDQ) {
        // P over the S columns this thread has just consumed, then hand it to the MMA warp
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) pk[i] = pack16x2<BF16>(p[cc * 32 + 2 * i], p[cc * 32 + 2 * i + 1]);
          tmem_st16(t_s + cc * 16, pk);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&sm.p_ready);
      }

      // ---- phase 2: dS = P * (dP - delta)
      if (threadIdx.x == 0) KB_TR(2, t, 2);
      ok = __all_sync(0xffffffffu, mbar_wait(&sm.dp_ready, t & 1, ctx, kWDpReady));
      if (!ok) break;
      if (threadIdx.x == 0) KB_TR(2, t, 3);
      tc_fence_after();
      {
        uint32_t dp[64];
        tmem_ld32(t_dp, reinterpret_cast<uint32_t(&)[32]>(dp[0]));
        tmem_ld32(t_dp + 32, reinterpret_cast<uint32_t(&)[32]>(dp[32]));
        tmem_wait_ld();
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            float4 dv = make_float4(delta_r, delta_r, delta_r, delta_r);
            if (!kDQ) dv = *reinterpret_cast<const float4*>(delta_c + cc * 32 + 2 * i);
            const int e = cc * 32 + 2 * i;
            pk[i] = pack16x2<BF16>(p[e] * (__uint_as_float(dp[e]) - dv.x), p[e + 1] * (__uint_as_float(dp[e + 1]) - dv.y));
            pk[i + 1] = pack16x2<BF16>(p[e + 2] * (__uint_as_float(dp[e + 2]) - dv.z), p[e + 3] * (__uint_as_float(dp[e + 3]) - dv.w));
          }
          tmem_st16(t_dp + cc * 16, pk);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&sm.ds_ready[t & 1]);
      if (threadIdx.x == 0) KB_TR(2, t, 4);
    }

    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&sm.acc_done, 0, ctx, kWAccDone));
    if (ok) {
      // Every MMA and every TMA load of this CTA is complete: the B1 ring is free and becomes the
      // staging area of the outputs (b1[0]: accumulator 1, b1[1]: accumulator 2), in the same
      // 64-column swizzled panels TMA expects, so that the rows leave as bulk tensor stores
      // instead of 16-byte stores scattered over 128 rows.
      tc_fence_after();
#pragma unroll
      for (int which = 0; which < (kDQ ? 1 : 2); ++which) {
        const uint32_t col0 = which == 0 ? kColAcc1 : kColAcc2;
        // dQ and dK carry the softmax scale; dV does not
        const float mul = (kDQ || which == 1) ? a.sm_scale : 1.f;
        uint8_t* stage = sm.b1[which];
#pragma unroll
        for (int cc = 0; cc < D / 64; ++cc) {
          const int c32 = half * (D / 64) + cc;  // this warpgroup's share of the D columns, 32 at a time
          uint32_t r[32];
          tmem_ld32(t_lane + col0 + c32 * 32, r);
          tmem_wait_ld();
          uint8_t* prow = stage + (c32 / 2) * kPanelBytes + row * 128;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack16x2<BF16>(__uint_as_float(r[8 * g + 0]) * mul, __uint_as_float(r[8 * g + 1]) * mul);
            w.y = pack16x2<BF16>(__uint_as_float(r[8 * g + 2]) * mul, __uint_as_float(r[8 * g + 3]) * mul);
            w.z = pack16x2<BF16>(__uint_as_float(r[8 * g + 4]) * mul, __uint_as_float(r[8 * g + 5]) * mul);
            w.w = pack16x2<BF16>(__uint_as_float(r[8 * g + 6]) * mul, __uint_as_float(r[8 * g + 7]) * mul);
            const int chunk = (c32 & 1) * 4 + g;  // 16-byte chunk within the 128-byte panel row
            *reinterpret_cast<uint4*>(prow + ((chunk ^ (row & 7)) << 4)) = w;
          }
        }
      }
      fence_proxy_async();
      mbar_arrive(&sm.staged);
      if (threadIdx.x == 0) {
        if (mbar_wait(&sm.staged, 0, ctx, kWStaged)) {
#pragma unroll
          for (int which = 0; which < (kDQ ? 1 : 2); ++which)
#pragma unroll
            for (int p = 0; p < kPanels; ++p)
              tma_store_4d(which == 0 ? &tm_out1 : &tm_out2, sm.b1[which] + p * kPanelBytes, p * 64, x0, h, b);
          tma_store_commit();
          tma_store_wait_all();
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    if (sm.abort_flag) __nanosleep(1000000);  // let copies still in flight land before the CTA goes away
    tmem_dealloc(tmem, kTmemCols);
  }
}

// The six tensor maps of one pass.  Both passes' maps are made before either pass is launched, so
// "unsupported" (a layout no map describes) always means that nothing ran.
struct PassMaps {
  CUtensorMap a1, a2, b1, b2, o1, o2;
};
template <int D, bool kDQ>
bool make_pass_maps(PassMaps* m, const kb_sa_bwd_params& p) {
  const kb_tensor4& a1 = kDQ ? p.q : p.k;
  const kb_tensor4& a2 = kDQ ? p.d_o : p.v;
  const kb_tensor4& b1 = kDQ ? p.k : p.q;
  const kb_tensor4& b2 = kDQ ? p.v : p.d_o;
  return make_tile_map_4d(&m->a1, a1, p.B, p.H, p.T, D, kBX) && make_tile_map_4d(&m->a2, a2, p.B, p.H, p.T, D, kBX) &&
         make_tile_map_4d(&m->b1, b1, p.B, p.H, p.T, D, kBY) && make_tile_map_4d(&m->b2, b2, p.B, p.H, p.T, D, kBY) &&
         make_tile_map_4d_contiguous(&m->o1, kDQ ? p.dq : p.dv, p.B, p.H, p.T, D, kBX) &&
         make_tile_map_4d_contiguous(&m->o2, kDQ ? p.dq : p.dk, p.B, p.H, p.T, D, kBX);
}

template <int D, bool BF16, bool kDQ>
int launch_pass(const kb_sa_bwd_params& p, const PassMaps& m, int32_t c, int32_t back, cudaStream_t s) {
  auto kern = sa_bwd_sm100_kernel<D, BF16, kDQ>;
  constexpr size_t smem = sizeof(BwdSmem<D>);
  static_assert(sizeof(BwdSmem<D>) <= 232448, "backward shared memory exceeds the 227 KB a CTA may have");
  int dev = 0, n_sm = 0;
  if (!device_sm_count(&dev, &n_sm)) return KB_ERR_LAUNCH;
  static std::atomic<bool> smem_opted_in[kMaxDevices];
  KB_CUDA_TRY(opt_in_smem_once(kern, smem, dev, smem_opted_in));
  BwdArgs a;
  a.o = static_cast<const uint16_t*>(p.o.data);
  a.d_o = static_cast<const uint16_t*>(p.d_o.data);
  a.o_sb = p.o.stride[0];
  a.o_sh = p.o.stride[1];
  a.o_st = p.o.stride[2];
  a.do_sb = p.d_o.stride[0];
  a.do_sh = p.d_o.stride[1];
  a.do_st = p.d_o.stride[2];
  a.lse = p.lse;
  a.delta = p.delta_ws;
  a.out1 = kDQ ? p.dq : p.dv;
  a.out2 = kDQ ? nullptr : p.dk;
  a.lens = p.lens;
  a.lens_stride = p.lens_stride;
  a.H = p.H;
  a.T = p.T;
  a.c = c;
  a.back = back;
  a.scale_log2 = p.sm_scale * kLog2e;
  a.sm_scale = p.sm_scale;
  a.status = p.status;
  dim3 grid(kb_cdiv_i32(p.T, kBX), p.H, p.B);
  kern<<<grid, kThreads, smem, s>>>(m.a1, m.a2, m.b1, m.b2, m.o1, m.o2, a);
  KB_LAUNCH_CHECK(kDQ ? "sa_bwd_sm100_kernel<dq>" : "sa_bwd_sm100_kernel<dkdv>");
  return KB_OK;
}

template <int D, bool BF16>
int launch_both(const kb_sa_bwd_params& p, int32_t c, int32_t back, cudaStream_t s) {
  const bool run_dq = !(p.flags & KB_FLAG_BWD_SKIP_DQ), run_dkdv = !(p.flags & KB_FLAG_BWD_SKIP_DKDV);
  PassMaps m_dq, m_dkdv;
  if ((run_dq && !make_pass_maps<D, true>(&m_dq, p)) || (run_dkdv && !make_pass_maps<D, false>(&m_dkdv, p)))
    return KB_ERR_UNSUPPORTED;
  if (run_dq) {
    const int rc = launch_pass<D, BF16, true>(p, m_dq, c, back, s);
    if (rc) return rc;
  }
  if (run_dkdv) {
    const int rc = launch_pass<D, BF16, false>(p, m_dkdv, c, back, s);
    if (rc) return rc;
  }
  return KB_OK;
}

}  // namespace

#ifdef KB_TRACE
}  // namespace kb
extern "C" __attribute__((visibility("default"))) int kb_debug_trace(long long* out) {
  return (int)cudaMemcpyFromSymbol(out, kb::g_trace, sizeof(kb::g_trace));
}
namespace kb {
#endif

int sa_bwd_sm100(const kb_sa_bwd_params& p, int32_t c, int32_t back, cudaStream_t s) {
  for (void* out : {p.dq, p.dk, p.dv})
    if (reinterpret_cast<uintptr_t>(out) % 16) return KB_ERR_UNSUPPORTED;
  // launch_both makes the tensor maps of both passes before it launches either, so "unsupported"
  // never leaves a half-finished backward behind
  const bool bf16 = p.dtype == KB_BF16;
  if (p.D == 64) return bf16 ? launch_both<64, true>(p, c, back, s) : launch_both<64, false>(p, c, back, s);
  if (p.D == 128) return bf16 ? launch_both<128, true>(p, c, back, s) : launch_both<128, false>(p, c, back, s);
  return KB_ERR_UNSUPPORTED;
}

}  // namespace kb
