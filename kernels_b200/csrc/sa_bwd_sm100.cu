// Streaming-attention backward for sm_100a: one kernel template, two passes.
//
//   dQ pass    (kDQ = true):  a CTA keeps 128 query rows (Q, dO) in shared memory and streams
//                             64-row K/V tiles over the forward schedule.  It also produces
//                             delta = rowsum(O * dO) for its rows and leaves it in the
//                             workspace for the other pass.
//   dK/dV pass (kDQ = false): a CTA keeps 128 key rows (K, V) and streams 64-row Q/dO tiles
//                             over the transposed schedule.
// Both passes have the same shape.  With X the stationary operands (A1, A2) and Y_t the
// streamed ones (B1, B2):
//   Z1 = A1 * B1^T   (scores, 128 x 64)          Z2 = A2 * B2^T   (dP, 128 x 64)
//   P  = 2^(Z1 * scale - lse[q])                 dS = P * (Z2 - delta[q])      (masked -> 0)
//   dQ pass:    dQ += dS * K_t                   dK/dV pass: dV += P * dO_t,  dK += dS * Q_t
// Z1/Z2 live in TMEM, double buffered; P and dS are written back over them as 16-bit values
// and feed the accumulating MMAs as the A operand straight from TMEM; the streamed tile in
// shared memory is read K-major by the first two MMAs and MN-major by the accumulating ones.
// The MMA warp issues Z(t+1) before the accumulation of tile t, so the tensor pipe works on
// one tile while the four compute warps turn the other tile's scores into P / dS.
//
// Roles: warps 0-7 compute (two warpgroups; a thread owns row (warp % 4) * 32 + lane = its TMEM
// lane, and warpgroup g the columns [32 g, 32 g + 32) of every 64-column tile), warp 8 TMA
// producer (plus the per-column lse/delta staging of the dK/dV pass), warp 9 MMA issuer and
// TMEM owner.
// TMEM columns: Z1[2] at 0/64, Z2[2] at 128/192, accumulator 1 at 256, accumulator 2 at 384.
//
// Reference semantics: src/streaming_attention/kernel.py:453-514 (delta), 639-773 and
// 941-1023 (dQ), 777-937 and 1027-1129 (dK/dV).  No atomics: results are bitwise repeatable.
#include <math.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "sm100_host.h"

namespace kb {
namespace {

using namespace sm100;

constexpr int kBX = 128;  // stationary rows per CTA
constexpr int kBY = 64;   // streamed rows per tile
constexpr int kStages = 4;
constexpr int kComputeWarps = 8;
constexpr int kThreads = (kComputeWarps + 2) * 32;
constexpr int kProducerWarp = kComputeWarps, kMmaWarp = kComputeWarps + 1;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColZ1 = 0, kColZ2 = 128, kColAcc1 = 256, kColAcc2 = 384;

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

template <int D>
struct alignas(1024) BwdSmem {
  uint8_t a1[kBX * D * 2];
  uint8_t a2[kBX * D * 2];
  uint8_t y1[kStages][kBY * D * 2];
  uint8_t y2[kStages][kBY * D * 2];
  alignas(16) float lse_s[kStages][kBY];
  alignas(16) float delta_s[kStages][kBY];
  uint64_t x_full, y_full[kStages], y_empty[kStages], z_ready[2], p_ready[2], z_free[2], acc_done;
  uint32_t tmem_base;
  int abort_flag;
};

enum WaitSite { kWX = 21, kWYEmpty, kWYFull, kWZFree, kWZReady, kWPReady, kWAccDone };

template <int D, bool BF16, bool kDQ, bool kWaitZFree>
__global__ void __launch_bounds__(kThreads, 1)
sa_bwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_a1, const __grid_constant__ CUtensorMap tm_a2,
                    const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_b2,
                    const BwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  BwdSmem<D>& sm = *reinterpret_cast<BwdSmem<D>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y, x0 = blockIdx.x * kBX;
  const int T = a.T;
  const int len = a.lens ? kb_clamp_len(a.lens[(int64_t)b * a.lens_stride], T) : T;
  const int64_t bh = (int64_t)b * a.H + h;
  uint16_t* out1 = static_cast<uint16_t*>(a.out1) + bh * T * D;
  uint16_t* out2 = kDQ ? nullptr : static_cast<uint16_t*>(a.out2) + bh * T * D;

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

  if (threadIdx.x == 0) {
    mbar_init(&sm.x_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sm.y_full[s], 1);
      mbar_init(&sm.y_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.z_ready[i], 1);
      mbar_init(&sm.p_ready[i], kComputeWarps * 32);
      mbar_init(&sm.z_free[i], 1);
    }
    mbar_init(&sm.acc_done, 1);
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
  constexpr uint32_t kXPanelBytes = kBX * 128, kYPanelBytes = kBY * 128;
  constexpr uint32_t kXBytes = kBX * D * 2, kYBytes = kBY * D * 2;

  if (warp == kProducerWarp) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&tm_a1);
      prefetch_tensormap(&tm_a2);
      prefetch_tensormap(&tm_b1);
      prefetch_tensormap(&tm_b2);
      mbar_expect_tx(&sm.x_full, 2 * kXBytes);
#pragma unroll
      for (int p = 0; p < kPanels; ++p) {
        tma_load_4d(sm.a1 + p * kXPanelBytes, &tm_a1, &sm.x_full, p * 64, x0, h, b);
        tma_load_4d(sm.a2 + p * kXPanelBytes, &tm_a2, &sm.x_full, p * 64, x0, h, b);
      }
    }
    for (int t = 0; t < n_tiles; ++t) {
      const int s = t % kStages;
      const int y0 = (yr.begin + t) * kBY;
      bool ok = true;
      if (t >= kStages) ok = mbar_wait(&sm.y_empty[s], ((t / kStages) - 1) & 1, ctx, kWYEmpty);
      if (!__all_sync(0xffffffffu, ok)) break;
      if (!kDQ) {
        // per-column statistics of the streamed query rows
#pragma unroll
        for (int i = 0; i < kBY / 32; ++i) {
          const int r = y0 + lane + 32 * i;
          const bool valid = r < len;
          sm.lse_s[s][lane + 32 * i] = valid ? a.lse[bh * T + r] : 0.f;
          sm.delta_s[s][lane + 32 * i] = valid ? a.delta[bh * T + r] : 0.f;
        }
        __syncwarp();
      }
      if (lane == 0) {
        mbar_expect_tx(&sm.y_full[s], 2 * kYBytes);
#pragma unroll
        for (int p = 0; p < kPanels; ++p) {
          tma_load_4d(sm.y1[s] + p * kYPanelBytes, &tm_b1, &sm.y_full[s], p * 64, y0, h, b);
          tma_load_4d(sm.y2[s] + p * kYPanelBytes, &tm_b2, &sm.y_full[s], p * 64, y0, h, b);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_z = make_idesc(BF16, kBX, kBY, false, false);
      constexpr uint32_t idesc_acc = make_idesc(BF16, kBX, D, false, true);
      const uint32_t a1_addr = smem_u32(sm.a1), a2_addr = smem_u32(sm.a2);
      bool ok = mbar_wait(&sm.x_full, 0, ctx, kWX);
      for (int t = 0; ok && t <= n_tiles; ++t) {
        if (t < n_tiles) {
          const int s = t % kStages, buf = t & 1;
          if (!mbar_wait(&sm.y_full[s], (t / kStages) & 1, ctx, kWYFull)) break;
          if (kWaitZFree && t >= 2 && !mbar_wait(&sm.z_free[buf], ((t / 2) - 1) & 1, ctx, kWZFree)) break;
          tc_fence_after();
          const uint32_t y1_addr = smem_u32(sm.y1[s]), y2_addr = smem_u32(sm.y2[s]);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t xo = (kk / 4) * kXPanelBytes + (kk % 4) * 32, yo = (kk / 4) * kYPanelBytes + (kk % 4) * 32;
            mma_ss(tmem + kColZ1 + buf * kBY, desc_kmajor(a1_addr + xo), desc_kmajor(y1_addr + yo), idesc_z, kk > 0);
          }
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t xo = (kk / 4) * kXPanelBytes + (kk % 4) * 32, yo = (kk / 4) * kYPanelBytes + (kk % 4) * 32;
            mma_ss(tmem + kColZ2 + buf * kBY, desc_kmajor(a2_addr + xo), desc_kmajor(y2_addr + yo), idesc_z, kk > 0);
          }
          mma_commit(&sm.z_ready[buf]);
        }
        if (t >= 1) {
          const int u = t - 1, s = u % kStages, buf = u & 1;
          if (!mbar_wait(&sm.p_ready[buf], (u / 2) & 1, ctx, kWPReady)) break;
          tc_fence_after();
          const uint32_t y1_addr = smem_u32(sm.y1[s]), y2_addr = smem_u32(sm.y2[s]);
          const uint32_t p_addr = tmem + kColZ1 + buf * kBY, ds_addr = tmem + kColZ2 + buf * kBY;
#pragma unroll
          for (int kk = 0; kk < kBY / 16; ++kk) {
            const bool acc = u > 0 || kk > 0;
            // 16 reduction rows = 8 packed columns; rows [32 g, 32 g + 32) sit at columns 32 g ..
            const uint32_t ko = (kk / 2) * 32 + (kk % 2) * 8;
            if (kDQ) {
              mma_ts(tmem + kColAcc1, ds_addr + ko, desc_mnmajor(y1_addr + kk * 2048, kYPanelBytes), idesc_acc, acc);
            } else {
              mma_ts(tmem + kColAcc1, p_addr + ko, desc_mnmajor(y2_addr + kk * 2048, kYPanelBytes), idesc_acc, acc);
              mma_ts(tmem + kColAcc2, ds_addr + ko, desc_mnmajor(y1_addr + kk * 2048, kYPanelBytes), idesc_acc, acc);
            }
          }
          mma_commit(&sm.y_empty[s]);
          mma_commit(&sm.z_free[buf]);
          if (u == n_tiles - 1) mma_commit(&sm.acc_done);
        }
      }
    }
  } else {
    // ------------------------------ compute warps + epilogue ------------------------------
    const int row = (warp & 3) * 32 + lane;
    const int half = warp >> 2;  // which 32 columns of each 64-column tile this warpgroup owns
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
    if (kDQ) {
      if (xi < len) {
        const uint4* orow = reinterpret_cast<const uint4*>(a.o + b * a.o_sb + h * a.o_sh + (int64_t)xi * a.o_st);
        const uint4* grow = reinterpret_cast<const uint4*>(a.d_o + b * a.do_sb + h * a.do_sh + (int64_t)xi * a.do_st);
        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int i = 0; i < D * 2 / 16; ++i) {
          const uint4 ov = __ldg(orow + i), gv = __ldg(grow + i);
          const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
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
            part[w] = fmaf(o0, g0, part[w]);
            part[w] = fmaf(o1, g1, part[w]);
          }
        }
        delta_r = (part[0] + part[1]) + (part[2] + part[3]);
        lse_r = a.lse[bh * T + xi];
      }
      if (half == 0 && xi < T) a.delta[bh * T + xi] = delta_r;
    }

    bool ok = true;
    for (int t = 0; t < n_tiles; ++t) {
      const int s = t % kStages, buf = t & 1;
      const int y0 = (yr.begin + t) * kBY + half * 32;  // first column this thread handles
      ok = __all_sync(0xffffffffu, mbar_wait(&sm.z_ready[buf], (t / 2) & 1, ctx, kWZReady));
      if (!ok) break;
      tc_fence_after();
      const bool warp_full = __all_sync(0xffffffffu, lo <= y0 && y0 + 32 <= hi);
      const uint32_t t_z1 = t_lane + kColZ1 + buf * kBY, t_z2 = t_lane + kColZ2 + buf * kBY;
      uint32_t z1[32], z2[32];
      tmem_ld32(t_z1 + half * 32, z1);
      tmem_ld32(t_z2 + half * 32, z2);
      float lse_c[32], delta_c[32];
      if (!kDQ) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 lv = *reinterpret_cast<const float4*>(&sm.lse_s[s][half * 32 + 4 * i]);
          const float4 dv = *reinterpret_cast<const float4*>(&sm.delta_s[s][half * 32 + 4 * i]);
          lse_c[4 * i] = lv.x, lse_c[4 * i + 1] = lv.y, lse_c[4 * i + 2] = lv.z, lse_c[4 * i + 3] = lv.w;
          delta_c[4 * i] = dv.x, delta_c[4 * i + 1] = dv.y, delta_c[4 * i + 2] = dv.z, delta_c[4 * i + 3] = dv.w;
        }
      }
      tmem_wait_ld();
      uint32_t pk_p[16], pk_ds[16];
      if (warp_full) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(z1[i]), scale, -(kDQ ? lse_r : lse_c[i])));
          const float p1 = ex2_approx(fmaf(__uint_as_float(z1[i + 1]), scale, -(kDQ ? lse_r : lse_c[i + 1])));
          const float d0 = p0 * (__uint_as_float(z2[i]) - (kDQ ? delta_r : delta_c[i]));
          const float d1 = p1 * (__uint_as_float(z2[i + 1]) - (kDQ ? delta_r : delta_c[i + 1]));
          if (!kDQ) pk_p[i / 2] = pack16x2<BF16>(p0, p1);
          pk_ds[i / 2] = pack16x2<BF16>(d0, d1);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ex2_approx(fmaf(__uint_as_float(z1[i]), scale, -(kDQ ? lse_r : lse_c[i])));
          float p1 = ex2_approx(fmaf(__uint_as_float(z1[i + 1]), scale, -(kDQ ? lse_r : lse_c[i + 1])));
          p0 = (y0 + i >= lo && y0 + i < hi) ? p0 : 0.f;
          p1 = (y0 + i + 1 >= lo && y0 + i + 1 < hi) ? p1 : 0.f;
          const float d0 = p0 * (__uint_as_float(z2[i]) - (kDQ ? delta_r : delta_c[i]));
          const float d1 = p1 * (__uint_as_float(z2[i + 1]) - (kDQ ? delta_r : delta_c[i + 1]));
          if (!kDQ) pk_p[i / 2] = pack16x2<BF16>(p0, p1);
          pk_ds[i / 2] = pack16x2<BF16>(d0, d1);
        }
      }
      // each warpgroup overlays its 16-bit values on the fp32 columns it has just consumed itself
      // (columns [32 g, 32 g + 16) of the buffer), so the two warpgroups never touch each other's data
      if (!kDQ) tmem_st16(t_z1 + half * 32, pk_p);
      tmem_st16(t_z2 + half * 32, pk_ds);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&sm.p_ready[buf]);
    }

    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&sm.acc_done, 0, ctx, kWAccDone));
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int which = 0; which < (kDQ ? 1 : 2); ++which) {
        const uint32_t col0 = which == 0 ? kColAcc1 : kColAcc2;
        // dQ and dK carry the softmax scale; dV does not
        const float mul = (kDQ || which == 1) ? a.sm_scale : 1.f;
        uint16_t* out = which == 0 ? out1 : out2;
#pragma unroll
        for (int cc = 0; cc < D / 64; ++cc) {
          const int c32 = half * (D / 64) + cc;  // this warpgroup's share of the D columns
          uint32_t r[32];
          tmem_ld32(t_lane + col0 + c32 * 32, r);
          tmem_wait_ld();
          if (xi < T) {
            uint4* dst = reinterpret_cast<uint4*>(out + (int64_t)xi * D + c32 * 32);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 w;
              w.x = pack16x2<BF16>(__uint_as_float(r[8 * g + 0]) * mul, __uint_as_float(r[8 * g + 1]) * mul);
              w.y = pack16x2<BF16>(__uint_as_float(r[8 * g + 2]) * mul, __uint_as_float(r[8 * g + 3]) * mul);
              w.z = pack16x2<BF16>(__uint_as_float(r[8 * g + 4]) * mul, __uint_as_float(r[8 * g + 5]) * mul);
              w.w = pack16x2<BF16>(__uint_as_float(r[8 * g + 6]) * mul, __uint_as_float(r[8 * g + 7]) * mul);
              dst[g] = w;
            }
          }
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

template <int D, bool BF16, bool kDQ>
int launch_pass(const kb_sa_bwd_params& p, int32_t c, int32_t back, cudaStream_t s) {
  CUtensorMap tm_a1, tm_a2, tm_b1, tm_b2;
  const kb_tensor4& a1 = kDQ ? p.q : p.k;
  const kb_tensor4& a2 = kDQ ? p.d_o : p.v;
  const kb_tensor4& b1 = kDQ ? p.k : p.q;
  const kb_tensor4& b2 = kDQ ? p.v : p.d_o;
  if (!make_tile_map_4d(&tm_a1, a1, p.B, p.H, p.T, D, kBX) || !make_tile_map_4d(&tm_a2, a2, p.B, p.H, p.T, D, kBX) ||
      !make_tile_map_4d(&tm_b1, b1, p.B, p.H, p.T, D, kBY) || !make_tile_map_4d(&tm_b2, b2, p.B, p.H, p.T, D, kBY))
    return KB_ERR_UNSUPPORTED;
  constexpr bool kWaitZFree = false;
  auto kern = sa_bwd_sm100_kernel<D, BF16, kDQ, kWaitZFree>;
  constexpr size_t smem = sizeof(BwdSmem<D>) + 1024;
  KB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
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
  kern<<<grid, kThreads, smem, s>>>(tm_a1, tm_a2, tm_b1, tm_b2, a);
  KB_LAUNCH_CHECK(kDQ ? "sa_bwd_sm100_kernel<dq>" : "sa_bwd_sm100_kernel<dkdv>");
  return KB_OK;
}

template <int D, bool BF16>
int launch_both(const kb_sa_bwd_params& p, int32_t c, int32_t back, cudaStream_t s) {
  if (!(p.flags & KB_FLAG_BWD_SKIP_DQ)) {
    const int rc = launch_pass<D, BF16, true>(p, c, back, s);
    if (rc) return rc;
  }
  if (!(p.flags & KB_FLAG_BWD_SKIP_DKDV)) {
    const int rc = launch_pass<D, BF16, false>(p, c, back, s);
    if (rc) return rc;
  }
  return KB_OK;
}

}  // namespace

int sa_bwd_sm100(const kb_sa_bwd_params& p, int32_t c, int32_t back, cudaStream_t s) {
  for (void* out : {p.dq, p.dk, p.dv})
    if (reinterpret_cast<uintptr_t>(out) % 16) return KB_ERR_UNSUPPORTED;
  // tensor maps are built before anything is launched, so "unsupported" never leaves a
  // half-finished backward behind
  const bool bf16 = p.dtype == KB_BF16;
  if (p.D == 64) return bf16 ? launch_both<64, true>(p, c, back, s) : launch_both<64, false>(p, c, back, s);
  if (p.D == 128) return bf16 ? launch_both<128, true>(p, c, back, s) : launch_both<128, false>(p, c, back, s);
  return KB_ERR_UNSUPPORTED;
}

}  // namespace kb
