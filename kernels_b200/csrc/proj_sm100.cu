// The two projections on either side of the attention operator, as sm_100a GEMMs that read and write
// the attention kernels' own tensor layout:
//   * QKV projection with rotary position embedding (kb_qkv_rope_proj): x [B, T, E] times the stacked
//     weight [(H + 2 H_kv) D, E] gives q [B, H, T, D], k and v [B, H_kv, T, D]; the rotation of q and k is
//     applied to the fp32 accumulator, so q, k, v are written once, already in the layout the attention
//     forward's tensor maps read (no [B, T, 3, H, D] intermediate, no transpose, no separate RoPE pass);
//   * output projection (kb_out_proj): o [B, H, T, D] (any strides the tensor maps take: the heads are
//     walked by the reduction loop) times w [E_out, H D] gives y [B, T, E_out].
// The reference project has neither (its callers run torch.nn.Linear around the operator); the seam is its
// public call, src/streaming_attention/kernel.py:1599-1652 (inputs q, k, v [B, H, T, D], output O).
//
// One kernel template, run by CTA pairs (clusters of 2, `tcgen05.mma.cta_group::2`).  A pair's tile is 256 tokens x
// 256 output features: CTA r of the pair owns tokens [128 r, 128 r + 128) of it (its A rows, its accumulator rows,
// its epilogue) and brings in half of the weight tile (feature rows [128 r, 128 r + 128)); the M256 N256 K16
// instruction, issued by one thread of the pair's leader, takes 128 clocks on each SM, so that thread keeps both
// tensor pipes fed with room to spare, and each SM fetches 8 KB of operands per instruction from its shared memory
// instead of the 12 KB a single-CTA M128 N256 instruction needs.  The reduction runs in steps of 64 elements (one
// 128-byte swizzled panel per row): per step each CTA's producer brings its 16 KB activation tile and its 16 KB half of
// the weight tile into a six-stage ring with TMA, the peer's MMA warp forwards "my tiles of this stage have
// landed" to the leader's barrier, and the leader's MMA thread issues four instructions; its commits arrive on
// the barriers of both CTAs.  The fp32 accumulator (256 TMEM columns in each CTA) is double buffered, so the four
// epilogue warps of each CTA (thread = token row = TMEM lane) convert, rotate, stage and TMA-store a finished
// tile while the next one is being accumulated.  Persistent: one pair per two SMs walks the tiles, feature tiles
// fastest, so pairs running at the same time share activation tiles in L2 (the weight is read once per wave and
// stays in L2).  Bound: tensor pipe.
//
// Rotary embedding, "rotate half" convention: for a head's element pair (d, d + D/2) at position t
//   out[d] = a[d] cos(t, d) - a[d + D/2] sin(t, d),   out[d + D/2] = a[d + D/2] cos(t, d) + a[d] sin(t, d),
// with cos / sin given as fp32 tables [D/2, T] (frequency-major: the 32 lanes of a warp, one token row
// each, read consecutive addresses).
#include <math.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "sm100_host.h"

namespace kb {
namespace {

using namespace sm100;

constexpr int kPM = 128;  // tokens per tile
constexpr int kPN = 256;  // output features per tile
constexpr int kPK = 64;   // reduction elements per stage
constexpr int kPStages = 6;
constexpr int kPThreads = 192;
constexpr int kPProducerWarp = 4, kPMmaWarp = 5;
constexpr uint32_t kPTmemCols = 512;  // two accumulators of 256 columns
constexpr uint32_t kPATileBytes = kPM * kPK * 2, kPBTileBytes = (kPN / 2) * kPK * 2;  // per CTA: its tokens, its half of the features
constexpr uint32_t kPPanelBytes = 128 * 128;  // 128 rows x 128 bytes

struct ProjArgs {
  int32_t B, T;             // batch entries, tokens per entry
  int32_t n_mt, n_nt;       // token tiles OF A PAIR (256 tokens) per batch entry, feature tiles
  int32_t k_steps;          // reduction steps of 64 elements
  int32_t a_inner_steps;    // steps per A "head": E / 64 for x, D / 64 for o (the A map's third coordinate counts heads)
  // output: feature tile nt covers features [256 nt, 256 nt + 256) = 256 / D heads of the stacked q | k | v
  // weight (D = 0: plain output y, features are columns)
  int32_t D, H, Hk;
  const float* rope_cos;  // [D / 2, T] or NULL
  const float* rope_sin;
  KbFastDiv fd_nt, fd_mt;
  int32_t* status;
};

struct alignas(1024) ProjSmem {
  uint8_t a[kPStages][kPATileBytes];
  uint8_t b[kPStages][kPBTileBytes];
  uint8_t out[2 * kPPanelBytes];  // 128 rows x 128 columns of output on their way to TMA stores
  uint64_t full[kPStages], empty[kPStages], acc_done[2], acc_free[2];
  uint32_t tmem_base;
  int abort_flag;
};

enum WaitSite { kWPEmpty = 101, kWPFull, kWPAccFree, kWPAccDone, kWPForward };
constexpr int kErrSmemAlign = 111;

template <bool BF16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPThreads, 1)
proj_sm100_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                  const __grid_constant__ CUtensorMap tm_o0, const __grid_constant__ CUtensorMap tm_o1,
                  const __grid_constant__ CUtensorMap tm_o2, const ProjArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  ProjSmem& sm = *reinterpret_cast<ProjSmem*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_items = a.B * a.n_mt * a.n_nt;
  const uint32_t rank = cluster_ctarank();              // 0: the pair's leader
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (smem_u32(smem_raw) & 1023u) {  // (the same in both CTAs of a pair)
    if (threadIdx.x == 0 && a.status) {
      atomicExch(a.status, KB_ERR_DEVICE_TIMEOUT);
      atomicExch(a.status + 1, kErrSmemAlign);
    }
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kPStages; ++s) {
      // the leader's: its own producer (with the bytes of its two tiles) and the peer's forwarded arrival
      mbar_init(&sm.full[s], rank == 0 ? 2 : 1);
      mbar_init(&sm.empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.acc_done[i], 1);
      mbar_init(&sm.acc_free[i], 256);  // the leader's is the one used: the epilogue threads of both CTAs arrive on it
    }
    sm.abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (warp == kPMmaWarp) tmem_alloc_pair(&sm.tmem_base, kPTmemCols);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before either arrives on the other's
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const WaitCtx ctx{&sm.abort_flag, a.status};

  // item -> (batch entry, token tile of the pair, feature tile), feature tile fastest
  auto decode = [&](int item, int& b, int& mt, int& nt) {
    const int bm = kb_fastdiv(item, a.fd_nt);
    nt = item - bm * a.n_nt;
    b = kb_fastdiv(bm, a.fd_mt);
    mt = 2 * (bm - b * a.n_mt) + (int)rank;  // this CTA's tile of 128 tokens
  };

  if (warp == kPProducerWarp) {
    if (lane == 0) {
      prefetch_tensormap(&tm_a);
      prefetch_tensormap(&tm_b);
      int u = 0;  // stages filled so far
      bool ok = true;
      for (int item = pair; ok && item < n_items; item += n_pairs) {
        int b, mt, nt;
        decode(item, b, mt, nt);
        int inner = 0, head = 0;  // position of the step inside A: element 64 * inner of "head" `head`
        for (int kk = 0; kk < a.k_steps; ++kk, ++u) {
          const int s = u % kPStages;
          if (u >= kPStages && !mbar_wait(&sm.empty[s], ((u / kPStages) - 1) & 1, ctx, kWPEmpty)) { ok = false; break; }
          mbar_expect_tx(&sm.full[s], kPATileBytes + kPBTileBytes);
          tma_load_4d(sm.a[s], &tm_a, &sm.full[s], inner * kPK, mt * kPM, head, b);
          tma_load_4d(sm.b[s], &tm_b, &sm.full[s], kk * kPK, nt * kPN + (int)rank * (kPN / 2), 0, 0);
          if (++inner == a.a_inner_steps) {
            inner = 0;
            ++head;
          }
        }
      }
    }
  } else if (warp == kPMmaWarp) {
    if (lane == 0 && rank == 0) {
      // ------------------------------ MMA issuer (leader) ------------------------------
      constexpr uint32_t idesc = make_idesc(BF16, 2 * kPM, kPN, false, false);
      int u = 0, m = 0;  // stages consumed, tiles so far
      bool ok = true;
      for (int item = pair; ok && item < n_items; item += n_pairs, ++m) {
        const uint32_t acc = tmem + (uint32_t)(m & 1) * kPN;
        if (m >= 2 && !mbar_wait(&sm.acc_free[m & 1], ((m >> 1) - 1) & 1, ctx, kWPAccFree)) break;
        tc_fence_after();
        for (int kk = 0; kk < a.k_steps; ++kk, ++u) {
          const int s = u % kPStages;
          if (!mbar_wait(&sm.full[s], (u / kPStages) & 1, ctx, kWPFull)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = desc_lo_kmajor(smem_u32(sm.a[s])), b_lo = desc_lo_kmajor(smem_u32(sm.b[s]));
#pragma unroll
          for (int i = 0; i < kPK / 16; ++i) mma_ss_lo_pair(acc, a_lo + 2 * i, b_lo + 2 * i, idesc, kk > 0 || i > 0);
          mma_commit_pair(&sm.empty[s]);
        }
        if (ok) mma_commit_pair(&sm.acc_done[m & 1]);
      }
    } else if (lane == 0) {
      // ------------------------------ peer: tiles landed -> the leader's barrier ------------------------------
      int u = 0;
      bool ok = true;
      for (int item = pair; ok && item < n_items; item += n_pairs) {
        for (int kk = 0; kk < a.k_steps; ++kk, ++u) {
          const int s = u % kPStages;
          if (!mbar_wait(&sm.full[s], (u / kPStages) & 1, ctx, kWPForward)) { ok = false; break; }
          mbar_arrive_cluster(&sm.full[s], 0);
        }
      }
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    const int row = warp * 32 + lane;
    const uint32_t t_lane = tmem + ((uint32_t)(warp * 32) << 16);
    const int D = a.D;
    int m = 0;
    bool ok = true;
    for (int item = pair; ok && item < n_items; item += n_pairs, ++m) {
      int b, mt, nt;
      decode(item, b, mt, nt);
      const int t = mt * kPM + row;  // this thread's token
      ok = named_barrier_and(1, 128, mbar_wait(&sm.acc_done[m & 1], (m >> 1) & 1, ctx, kWPAccDone));
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_acc = t_lane + (uint32_t)(m & 1) * kPN;
#pragma unroll 1
      for (int g = 0; g < kPN / 128; ++g) {  // 128 output columns at a time
        const int f0 = nt * kPN + g * 128;   // first feature of the group
        // which tensor and head the group goes to, and whether it is rotated
        int which = 0, head = 0;
        bool rope = false;
        if (D > 0) {
          head = f0 / D;
          if (head >= a.H + a.Hk) {
            which = 2;
            head -= a.H + a.Hk;
          } else if (head >= a.H) {
            which = 1;
            head -= a.H;
          }
          rope = a.rope_cos != nullptr && which < 2;
        }
        if (threadIdx.x == 0) tma_store_wait_read();  // the stores of the previous group have read the staging tile
        named_barrier_sync(2, 128);
        // two pairs of 32-column chunks: (lo, lo + D/2) with D = 128: lo = 0, 32; with D = 64: lo = 0, 64
        // (a plain projection is treated like D = 128 without rotation)
#pragma unroll 1
        for (int j = 0; j < 2; ++j) {
          const int lo = (D == 64) ? 64 * j : 32 * j, hi = lo + ((D == 64) ? 32 : 64);
          const int i0 = (D == 64) ? 0 : 32 * j;  // rotary index of the chunk's first element
          uint32_t x0[32], x1[32];
          tmem_ld32(t_acc + g * 128 + lo, x0);
          tmem_ld32(t_acc + g * 128 + hi, x1);
          tmem_wait_ld();
          if (g == kPN / 128 - 1 && j == 1) {
            tc_fence_before();
            mbar_arrive_cluster(&sm.acc_free[m & 1], 0);  // (the leader's barrier) the accumulator may be overwritten by the tile after next
          }
          if (rope && t < a.T) {
            const float* cs = a.rope_cos + (int64_t)i0 * a.T + t;
            const float* sn = a.rope_sin + (int64_t)i0 * a.T + t;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float c = __ldg(cs + (int64_t)i * a.T), s = __ldg(sn + (int64_t)i * a.T);
              const float u0 = __uint_as_float(x0[i]), u1 = __uint_as_float(x1[i]);
              x0[i] = __float_as_uint(u0 * c - u1 * s);
              x1[i] = __float_as_uint(u1 * c + u0 * s);
            }
          }
          // 32 columns = four 16-byte chunks of the row's 128-byte line in panel (column / 64)
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const uint32_t* x = half ? x1 : x0;
            const int col = half ? hi : lo;
            uint8_t* prow = sm.out + (col / 64) * kPPanelBytes + row * 128;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 w;
              w.x = pack16x2<BF16>(__uint_as_float(x[8 * q4 + 0]), __uint_as_float(x[8 * q4 + 1]));
              w.y = pack16x2<BF16>(__uint_as_float(x[8 * q4 + 2]), __uint_as_float(x[8 * q4 + 3]));
              w.z = pack16x2<BF16>(__uint_as_float(x[8 * q4 + 4]), __uint_as_float(x[8 * q4 + 5]));
              w.w = pack16x2<BF16>(__uint_as_float(x[8 * q4 + 6]), __uint_as_float(x[8 * q4 + 7]));
              const int chunk = (col % 64) / 8 + q4;
              *reinterpret_cast<uint4*>(prow + ((chunk ^ (row & 7)) << 4)) = w;
            }
          }
        }
        fence_proxy_async();
        named_barrier_sync(2, 128);
        if (threadIdx.x == 0 && mt * kPM < a.T) {  // (the second tile of a pair may lie wholly past the last token)
          const CUtensorMap* tm = which == 0 ? &tm_o0 : (which == 1 ? &tm_o1 : &tm_o2);
          if (D == 0) {
            // plain output [B, T, E_out]: the group's 128 columns are two 64-column boxes
            tma_store_4d(tm, sm.out, f0, mt * kPM, 0, b);
            tma_store_4d(tm, sm.out + kPPanelBytes, f0 + 64, mt * kPM, 0, b);
          } else if (D == 128) {
            tma_store_4d(tm, sm.out, 0, mt * kPM, head, b);
            tma_store_4d(tm, sm.out + kPPanelBytes, 64, mt * kPM, head, b);
          } else {  // D == 64: the group holds two heads, one per panel
            tma_store_4d(tm, sm.out, 0, mt * kPM, head, b);
            tma_store_4d(tm, sm.out + kPPanelBytes, 0, mt * kPM, head + 1, b);
          }
          tma_store_commit();
        }
      }
    }
    if (threadIdx.x == 0) tma_store_wait_all();
  }

  // neither CTA leaves, nor gives its TMEM back, while the other may still read its shared memory or arrive on
  // its barriers
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == kPMmaWarp) {
    if (sm.abort_flag) __nanosleep(1000000);  // let copies still in flight land before the CTA goes away
    tmem_dealloc_pair(tmem, kPTmemCols);
  }
}

// a contiguous row-major [rows, cols] 16-bit matrix as a kb_tensor4 with one batch entry and one head
kb_tensor4 matrix_view(const void* data, int64_t cols) {
  kb_tensor4 t;
  t.data = data;
  t.stride[0] = 0, t.stride[1] = 0, t.stride[2] = cols, t.stride[3] = 1;
  return t;
}

template <bool BF16>
int launch_proj(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& o0, const CUtensorMap& o1,
                const CUtensorMap& o2, const ProjArgs& a, cudaStream_t s) {
  auto kern = proj_sm100_kernel<BF16>;
  static_assert(sizeof(ProjSmem) <= 232448, "projection shared memory exceeds the 227 KB a CTA may have");
  int dev = 0, n_sm = 0;
  if (!device_sm_count(&dev, &n_sm)) return KB_ERR_LAUNCH;
  static std::atomic<bool> smem_opted_in[kMaxDevices];
  KB_CUDA_TRY(opt_in_smem_once(kern, sizeof(ProjSmem), dev, smem_opted_in));
  const int64_t n_items = (int64_t)a.B * a.n_mt * a.n_nt;
  if (n_items > (int64_t)1 << 30) return KB_ERR_TOO_LARGE;
  // Persistent: as many pairs as the device can hold at once (not every SM of a die can be paired up, so this
  // may be fewer than half the SM count; a grid larger than that would run its last pairs as a second wave).
  static std::atomic<int> pairs_cached[kMaxDevices];
  int max_pairs = pairs_cached[dev].load(std::memory_order_relaxed);
  if (max_pairs == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n_sm & ~1), 1, 1);
    cfg.blockDim = dim3(kPThreads, 1, 1);
    cfg.dynamicSmemBytes = sizeof(ProjSmem);
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2, attr.val.clusterDim.y = 1, attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) {
      (void)cudaGetLastError();
      n = n_sm / 2;
    }
    max_pairs = n < n_sm / 2 ? n : n_sm / 2;
    pairs_cached[dev].store(max_pairs, std::memory_order_relaxed);
  }
  const unsigned grid = 2u * (unsigned)(n_items < max_pairs ? n_items : max_pairs);
  kern<<<grid, kPThreads, sizeof(ProjSmem), s>>>(tm_a, tm_b, o0, o1, o2, a);
  KB_LAUNCH_CHECK("proj_sm100_kernel");
  return KB_OK;
}

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

}  // namespace
}  // namespace kb

extern "C" int kb_qkv_rope_proj(const kb_qkv_proj_params* p, void* stream) {
  using namespace kb;
  if (!p || p->B < 0 || p->T < 0 || p->E < 1 || p->H < 1 || p->H_kv < 1) return KB_ERR_BAD_ARGUMENT;
  if ((p->rope_cos == nullptr) != (p->rope_sin == nullptr)) return KB_ERR_BAD_ARGUMENT;
  if (p->dtype != KB_F16 && p->dtype != KB_BF16) return KB_ERR_UNSUPPORTED;
  if (p->D != 64 && p->D != 128) return KB_ERR_UNSUPPORTED;
  const int heads_per_tile = kPN / p->D;
  // a feature tile must hold whole heads of ONE of q, k, v, and the reduction runs in whole steps of 64
  if (p->H % heads_per_tile || p->H_kv % heads_per_tile || p->E % kPK) return KB_ERR_UNSUPPORTED;
  if (p->B == 0 || p->T == 0) return KB_OK;
  if (!p->x || !p->w || !p->q || !p->k || !p->v) return KB_ERR_BAD_ARGUMENT;
  for (const void* ptr : {p->x, p->w, (const void*)p->q, (const void*)p->k, (const void*)p->v})
    if (!aligned16(ptr)) return KB_ERR_UNSUPPORTED;
  const int64_t n_feat = (int64_t)(p->H + 2 * p->H_kv) * p->D;
  if (n_feat > (int64_t)1 << 30 || (int64_t)p->B * p->T > (int64_t)1 << 30) return KB_ERR_TOO_LARGE;

  CUtensorMap tm_a, tm_b, tm_q, tm_k, tm_v;
  kb_tensor4 xv;
  xv.data = p->x;
  xv.stride[0] = (int64_t)p->T * p->E, xv.stride[1] = 0, xv.stride[2] = p->E, xv.stride[3] = 1;
  const int64_t none[3] = {0, 0, 0};
  if (!make_tile_map_4d(&tm_a, xv, p->B, 1, p->T, p->E, kPM) ||
      !make_tile_map_4d(&tm_b, matrix_view(p->w, p->E), 1, 1, (int)n_feat, p->E, kPN / 2) ||
      !make_tile_map_4d(&tm_q, out_view(p->q, none, p->H, p->T, p->D), p->B, p->H, p->T, p->D, kPM) ||
      !make_tile_map_4d(&tm_k, out_view(p->k, none, p->H_kv, p->T, p->D), p->B, p->H_kv, p->T, p->D, kPM) ||
      !make_tile_map_4d(&tm_v, out_view(p->v, none, p->H_kv, p->T, p->D), p->B, p->H_kv, p->T, p->D, kPM))
    return KB_ERR_UNSUPPORTED;
  ProjArgs a;
  a.B = p->B, a.T = p->T;
  a.n_mt = kb_cdiv_i32(p->T, 2 * kPM);
  a.n_nt = (int32_t)(n_feat / kPN);
  a.k_steps = p->E / kPK;
  a.a_inner_steps = a.k_steps;
  a.D = p->D, a.H = p->H, a.Hk = p->H_kv;
  a.rope_cos = p->rope_cos, a.rope_sin = p->rope_sin;
  a.fd_nt = kb_fastdiv_make(a.n_nt), a.fd_mt = kb_fastdiv_make(a.n_mt);
  a.status = p->status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return p->dtype == KB_BF16 ? launch_proj<true>(tm_a, tm_b, tm_q, tm_k, tm_v, a, s)
                             : launch_proj<false>(tm_a, tm_b, tm_q, tm_k, tm_v, a, s);
}

extern "C" int kb_out_proj(const kb_out_proj_params* p, void* stream) {
  using namespace kb;
  if (!p || p->B < 0 || p->T < 0 || p->H < 1 || p->E_out < 1) return KB_ERR_BAD_ARGUMENT;
  if (p->dtype != KB_F16 && p->dtype != KB_BF16) return KB_ERR_UNSUPPORTED;
  if (p->D != 64 && p->D != 128) return KB_ERR_UNSUPPORTED;
  if (p->E_out % kPN) return KB_ERR_UNSUPPORTED;
  if (p->B == 0 || p->T == 0) return KB_OK;
  if (!p->o.data || !p->w || !p->y) return KB_ERR_BAD_ARGUMENT;
  if (!aligned16(p->w) || !aligned16(p->y)) return KB_ERR_UNSUPPORTED;
  if ((int64_t)p->H * p->D > (int64_t)1 << 30 || (int64_t)p->B * p->T > (int64_t)1 << 30) return KB_ERR_TOO_LARGE;

  CUtensorMap tm_a, tm_b, tm_y;
  kb_tensor4 yv;
  yv.data = p->y;
  yv.stride[0] = (int64_t)p->T * p->E_out, yv.stride[1] = 0, yv.stride[2] = p->E_out, yv.stride[3] = 1;
  if (!make_tile_map_4d(&tm_a, p->o, p->B, p->H, p->T, p->D, kPM) ||
      !make_tile_map_4d(&tm_b, matrix_view(p->w, (int64_t)p->H * p->D), 1, 1, p->E_out, p->H * p->D, kPN / 2) ||
      !make_tile_map_4d(&tm_y, yv, p->B, 1, p->T, p->E_out, kPM))
    return KB_ERR_UNSUPPORTED;
  ProjArgs a;
  a.B = p->B, a.T = p->T;
  a.n_mt = kb_cdiv_i32(p->T, 2 * kPM);
  a.n_nt = p->E_out / kPN;
  a.k_steps = p->H * p->D / kPK;
  a.a_inner_steps = p->D / kPK;
  a.D = 0, a.H = 0, a.Hk = 0;
  a.rope_cos = nullptr, a.rope_sin = nullptr;
  a.fd_nt = kb_fastdiv_make(a.n_nt), a.fd_mt = kb_fastdiv_make(a.n_mt);
  a.status = p->status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return p->dtype == KB_BF16 ? launch_proj<true>(tm_a, tm_b, tm_y, tm_y, tm_y, a, s)
                             : launch_proj<false>(tm_a, tm_b, tm_y, tm_y, tm_y, a, s);
}
