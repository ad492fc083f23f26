// Streaming-attention backward for sm_100a that computes the scores ONCE per (key tile, query tile)
// pair: five matmuls per pair instead of the seven a dQ pass plus a dK/dV pass execute, with no
// atomics or reductions in global memory (results are bitwise repeatable).
//
// Three launches:
//   1. delta   delta = rowsum(O * dO) per row;
//   2. main    persistent, one CTA per SM.  A work item is one tile of 128 key rows of one
//              (batch, head); the CTA keeps K and V of the item in shared memory and streams the
//              128-row Q / dO tiles of the transposed schedule (schedule.h).  Per tile pair
//                  S  = K Q^T            dP = V dO^T                 (keys x queries, into TMEM)
//                  P  = 2^(S scale - lse[q])       dS = P (dP - delta[q])        (masked -> 0)
//                  dV += P dO      dK += dS Q
//              dV and dK accumulate in TMEM over the item.  The 16-bit dS tile, which the dQ pass of
//              the two-pass kernels would have to recompute with two more matmuls, is kept: besides
//              TMEM (operand of dK) it is written to shared memory in the layout an MMA operand has
//              there and leaves for a scratch buffer in global memory as one 32 KB bulk copy;
//   3. dq      persistent.  A work item is one tile of 128 query rows; the CTA streams the saved dS
//              tiles of the forward schedule (bulk copies, straight into operand layout) with the
//              matching K tiles and accumulates dQ = sum_j dS_j^T K_j in TMEM: one matmul per pair.
// The dS scratch holds B * H * ceil(T/128) * W tiles of 32 KB, W = the most query tiles a key tile can
// meet (sa_bwd_fused_slots); problems whose scratch the caller cannot afford use the two-pass kernels.
//
// Main kernel, 16 warps:
//   warps 0-7   compute: thread = key row (TMEM lane), warpgroup w owns query columns [64 w, 64 w + 64)
//               of every tile.  Phase 1 turns S into P (16-bit, back into TMEM over S); phase 2
//               turns dP into dS (16-bit, into TMEM over dP and into shared memory);
//   warps 8-11  epilogue: end of item, dV and dK TMEM -> 16-bit -> shared memory -> TMA store;
//   warp 12     TMA producer (one lane);
//   warp 13     MMA issuer (one lane), owner of the TMEM allocation;
//   warp 14     one lane sends each dS tile to the scratch buffer;
//   warp 15     per-tile staging of lse / delta into shared memory (whole warp; a role of its own so that the
//               latency of its global loads never holds back the producer's next TMA load).
// MMA issue order in steady state, tile g:   dV(g)  S(g+1)  dK(g)  dP(g+1).  MMAs execute in issue
// order, which makes the overlays in TMEM safe without extra waits (S(g+1) overwrites P(g) after
// dV(g) has read it, dP(g+1) overwrites dS(g) after dK(g) has read it).
//   TMEM columns  [0,128) S / P     [128,256) dP / dS     [256,384) dV     [384,512) dK
// The pipeline runs across items: tile g+1 may belong to the next item (K is double buffered, V is
// released by the item's last dP), and the epilogue warps empty dV / dK of an item while the first
// S, dP and P of the next one are under way.  Nothing but the lse / delta rows is moved by thread
// loads or stores: such traffic shares the path the MMAs fetch their operands through and was
// measured to slow them down severely.
// Shared memory at D = 128: K 2 x 32 KB, V 32, Q 2 x 32, dO 32, dS 32 = 224 KB.  The K buffer of a
// finished item stages its dV / dK on their way out before the K of the item after next lands in it.
//
// Reference semantics: src/streaming_attention/kernel.py:453-514 (delta), 639-773 and 941-1023
// (dQ), 777-937 and 1027-1129 (dK/dV).
#include <math.h>

#include "common.cuh"
#include <type_traits>

#include "sm100_ptx.cuh"
#include "sm100_host.h"
#include "tiles.h"

namespace kb {
#ifdef KB_TRACE_FUSED
// Debug build only: clock64 stamps of one CTA's pipeline events, read back by kb_debug_trace_fused().
// [role: 0 producer, 1 MMA, 2 compute warp 0, 3 epilogue / dq kernel][tile][slot]
__device__ long long g_ftrace[4][64][8];
#define KB_FTR(role, t, slot)                                                   \
  do {                                                                          \
    if (blockIdx.x == 60 && (t) < 64) g_ftrace[role][t][slot] = clock64();      \
  } while (0)
#else
#define KB_FTR(role, t, slot) \
  do {                        \
  } while (0)
#endif
namespace {

using namespace sm100;

constexpr int kBK = tiles::kMainKeys;     // key rows of a key tile
constexpr int kBQ = tiles::kMainQueries;  // query rows of a query tile
static_assert(kBK == 128 && kBQ == 128 && tiles::kDqQueries == kBQ && tiles::kDqKeys == kBK && tiles::kMainStagesQ == 2 &&
                  tiles::kMainStagesK == 2,
              "the TMEM column map, the dS tile layout and the buffer indexing assume 128 x 128 tiles and double buffers");
constexpr int kThreads = 512;
constexpr int kComputeThreads = 256, kEpiThreads = 128;
constexpr int kEpiWarp0 = 8, kProducerWarp = 12, kMmaWarp = 13, kSpillWarp = 14, kStatsWarp = 15;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kRelaxedNs = 0;  // poll interval of the roles off the critical chain (no gain measured from sleeping)
constexpr uint32_t kColS = 0, kColDP = 128, kColDV = 256, kColDK = 384;
// register budgets after the warpgroups have traded (launch budget: 128 per thread)
constexpr int kRegsCompute = 176, kRegsEpi = 104, kRegsOther = 56;
constexpr uint32_t kDsTileBytes = kBK * kBQ * 2;  // one dS tile: 2 panels x 128 key rows x 64 queries, 16-bit
constexpr uint32_t kPanelBytes = 128 * 128;       // 128 rows x 128 bytes

struct FusedArgs {
  const float* lse;
  const float* delta;
  uint8_t* ds_ws;  // dS scratch: tile (b, h, key tile kt, slot s) at (((b H + h) n_ktiles + kt) W + s) * 32 KB
  void* dk;        // written through tensor maps; the pointers serve key tiles that lie wholly in the padding
  void* dv;
  void* dq;
  const int32_t* lens;
  int64_t lens_stride;
  int64_t lse_sb, lse_sh;                      // element strides of lse (b, h)
  int64_t dq_sb, dq_sh, dq_st, dkv_sb, dkv_sh, dkv_st;  // of dq and of dk / dv (b, h, t)
  int32_t B, H, T, c, back, W;
  int32_t Hk, group;  // key/value heads and query heads per key/value head (H = Hk * group)
  // Packed batch: sequence b owns the rows [cu[b], cu[b + 1]) of tensors with ONE batch entry (the maps' batch
  // extent is 1, every *_sb stride is 0), T is the longest sequence, lse and delta are [H, total rows], and the
  // dS scratch is indexed by packed key tile (ptile_id below), n_ptiles of them per head.  NULL: padded layout.
  const int32_t* cu;
  int32_t total, n_ptiles;
  KbFastDiv fd_tiles, fd_H, fd_Hk, fd_group, fd_c;  // division by ceil(T / 128), H, Hk, group and c
  float scale_log2, sm_scale;
  int32_t* status;
};

// Most query tiles any key tile meets (the schedule with len = T; a shorter sequence only clips it).
inline int32_t fused_slots(int32_t T, int32_t c, int32_t back) {
  int32_t w = 1;
  for (int32_t k0 = 0; k0 < T; k0 += kBK) {
    const KbTileRange r = kb_bwd_q_range(k0, kBQ, kBK, T, c, back);
    w = kb_max_i32(w, r.end - r.begin);
  }
  return w;
}

// Upper bound on the key tiles of a packed batch (see ptile_id): every sequence may end one tile later than
// its rows alone would need.
inline int32_t packed_tiles(int32_t total, int32_t B) { return total / kBK + B + 1; }

template <int D>
struct alignas(1024) FusedSmem {
  uint8_t k[2][kBK * 128 * 2];  // 32 KB each whatever D is: they double as staging for dV / dK
  uint8_t v[kBK * D * 2];
  uint8_t q[2][kBQ * D * 2];
  uint8_t d_o[kBQ * D * 2];
  uint8_t ds[kDsTileBytes];  // rows = keys, 64 queries per 128-byte row, two panels
  alignas(16) float lse_s[2][kBQ];
  alignas(16) float delta_s[2][kBQ];
  uint64_t k_full[2], k_free[2], v_full, v_empty, q_full[2], q_empty[2], do_full, do_empty;
  uint64_t s_ready, p_ready, dp_ready, ds_ready[2], ds_free, stats_full[2], dv_done, dk_done, dv_free, dk_free;
  uint32_t tmem_base;
  int abort_flag;
};

enum WaitSite {
  kWKFree = 51, kWVEmpty, kWQEmpty, kWDoEmpty, kWStatsSlot, kWKFull, kWVFull, kWQFull, kWDoFull, kWPReady, kWAccFree,
  kWDsReady, kWSReady, kWStatsFull, kWDpReady, kWDsFree, kWAccDone, kWSpill,
  kWDqFull = 81, kWDqEmpty, kWDqAccDone, kWDqAccFree
};
constexpr int kErrSmemAlign = 71;

// One work item of the main kernel and the position of a tile in the CTA's tile sequence.  Every
// role walks the same sequence with its own cursor: `n` counts the live items so far, `g` the tiles
// so far; barrier phases are derived from them.
struct Item {
  int b, hk, kt, k0, len;  // hk: key/value head
  int row0;                // first row of the sequence in the tensor maps (packed batch: cu[b]; else 0)
  KbTileRange qr;          // query tiles [begin, end) of 128 rows that send gradient to this key tile
};
// The tiles of an item: for every query head of the key/value head's group (hq = 0 .. group - 1), the
// query tiles of `qr` (tq = 0 ..); t is the running index over both.
struct Cursor {
  int item, n, g, t, tq, hq, group;
  Item it;
  bool valid;
  __device__ __forceinline__ int q_tiles() const { return it.qr.end - it.qr.begin; }
  __device__ __forceinline__ int tiles() const { return group * q_tiles(); }
  __device__ __forceinline__ bool last() const { return t == tiles() - 1; }
  __device__ __forceinline__ int head() const { return it.hk * group + hq; }       // query head of the tile
  __device__ __forceinline__ int q0() const { return (it.qr.begin + tq) * kBQ; }   // its first query row
};

// `prev` is the item decoded before (b = -1: none): consecutive items mostly share the batch index
// and with it the sequence length, which saves the global load.
template <bool PACKED>
__device__ __forceinline__ Item decode_item(const FusedArgs& a, int item, int n_ktiles, const Item& prev) {
  Item it;
  const int bh = kb_fastdiv(item, a.fd_tiles);
  it.kt = item - bh * n_ktiles;
  it.b = kb_fastdiv(bh, a.fd_Hk);
  it.hk = bh - it.b * a.Hk;
  it.k0 = it.kt * kBK;
  it.row0 = 0;
  if (PACKED) {
    if (it.b == prev.b) {
      it.row0 = prev.row0;
      it.len = prev.len;
    } else {
      it.row0 = a.cu[it.b];
      it.len = kb_min_i32(a.cu[it.b + 1] - it.row0, a.T);
    }
  } else {
    it.len = !a.lens ? a.T : (it.b == prev.b ? prev.len : kb_clamp_len(a.lens[(int64_t)it.b * a.lens_stride], a.T));
  }
  it.qr = kb_bwd_q_range_fd(it.k0, kBQ, kBK, it.len, a.c, a.back, a.fd_c);
  return it;
}
// Packed batch: the number a key tile has among all key tiles of all sequences.  Sequence b starts at row
// row0 and is b-th in the batch; floor(row0 / 128) + b + kt is unique per (b, kt) and below
// floor(total / 128) + B + 1 (a sequence ends at most one tile later than its rows alone would need).
__device__ __forceinline__ int ptile_id(int row0, int b, int kt) { return (row0 >> 7) + b + kt; }
// first live item at or after `item` (stride gridDim.x)
template <bool PACKED>
__device__ __forceinline__ void seek_live(const FusedArgs& a, Cursor& c, int n_items, int n_ktiles) {
  c.valid = false;
  for (; c.item < n_items; c.item += gridDim.x) {
    c.it = decode_item<PACKED>(a, c.item, n_ktiles, c.it);
    if (c.it.qr.begin < c.it.qr.end) {
      c.valid = true;
      return;
    }
  }
}
template <bool PACKED>
__device__ __forceinline__ Cursor cursor_first(const FusedArgs& a, int n_items, int n_ktiles) {
  Cursor c;
  c.item = blockIdx.x;
  c.n = c.g = c.t = c.tq = c.hq = 0;
  c.group = a.group;
  c.it.b = -1;
  seek_live<PACKED>(a, c, n_items, n_ktiles);
  return c;
}
template <bool PACKED>
__device__ __forceinline__ void cursor_next(const FusedArgs& a, Cursor& c, int n_items, int n_ktiles) {
  ++c.g;
  ++c.t;
  if (++c.tq < c.q_tiles()) return;
  c.tq = 0;
  if (++c.hq < c.group) return;
  c.hq = 0;
  c.t = 0;
  ++c.n;
  c.item += gridDim.x;
  seek_live<PACKED>(a, c, n_items, n_ktiles);
}
// `h` is the QUERY head, `row0` the sequence's first row (packed batch only)
template <bool PACKED>
__device__ __forceinline__ uint8_t* ds_slot(const FusedArgs& a, int b, int row0, int h, int kt, int n_ktiles, int slot) {
  if (PACKED) return a.ds_ws + (((int64_t)h * a.n_ptiles + ptile_id(row0, b, kt)) * a.W + slot) * (int64_t)kDsTileBytes;
  return a.ds_ws + ((((int64_t)b * a.H + h) * n_ktiles + kt) * a.W + slot) * (int64_t)kDsTileBytes;
}

// PACKED: one launch over a packed batch (FusedArgs::cu).  MID: the MMA thread runs every tile through a copy of its
// issue sequence that has "opens its work item" and "closes it" compiled in, four copies in all (the class of long
// items of fully live tiles: head dim 128, chunks of 128 rows or more; 3-5 % on its main kernel, most of it from the
// copy for the tiles that do neither).  The other classes measured 3-12 % SLOWER with more than one copy in the
// kernel (shorter items: the rarely run copies fall out of the instruction cache), so they are built with one.
template <int D, bool BF16, bool PACKED, bool MID>
__global__ void __launch_bounds__(kThreads, 1)
sa_bwd_fused_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                    const FusedArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  FusedSmem<D>& sm = *reinterpret_cast<FusedSmem<D>*>(smem_raw);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T = a.T;
  const int n_ktiles = kb_cdiv_i32(T, kBK);
  const int n_items = a.B * a.Hk * n_ktiles;

  if (smem_u32(smem_raw) & 1023u) {
    // swizzled operand tiles need a 1024-byte aligned base: report instead of computing garbage
    if (threadIdx.x == 0 && a.status) {
      atomicExch(a.status, KB_ERR_DEVICE_TIMEOUT);
      atomicExch(a.status + 1, kErrSmemAlign);
    }
    return;
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.k_full[i], 1);
      mbar_init(&sm.k_free[i], 1);
      mbar_init(&sm.q_full[i], 1);
      mbar_init(&sm.q_empty[i], 1);
      mbar_init(&sm.ds_ready[i], kComputeThreads);
      mbar_init(&sm.stats_full[i], 32);
    }
    mbar_init(&sm.v_full, 1);
    mbar_init(&sm.v_empty, 1);
    mbar_init(&sm.do_full, 1);
    mbar_init(&sm.do_empty, 1);
    mbar_init(&sm.s_ready, 1);
    mbar_init(&sm.p_ready, kComputeThreads);
    mbar_init(&sm.dp_ready, 1);
    mbar_init(&sm.ds_free, 1);
    mbar_init(&sm.dv_done, 1);
    mbar_init(&sm.dk_done, 1);
    mbar_init(&sm.dv_free, kEpiThreads);
    mbar_init(&sm.dk_free, kEpiThreads);
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
  constexpr uint32_t kTileBytes = 128 * D * 2;
#ifdef KB_TRACE_FUSED
  if (threadIdx.x == 0 && blockIdx.x == 60) {
    g_ftrace[3][63][0] = clock64();
    g_ftrace[3][63][1] = (long long)globaltimer_ns();
  }
#endif

  if (warp >= kProducerWarp) {
    setmaxnreg_dec<kRegsOther>();
    if (warp == kProducerWarp) {
      // ------------------------------ TMA producer ------------------------------
      if (lane == 0) {
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_do);
      }
      bool ok = true;
      for (Cursor c = cursor_first<PACKED>(a, n_items, n_ktiles); ok && c.valid; cursor_next<PACKED>(a, c, n_items, n_ktiles)) {
        const int g = c.g, n = c.n;
        const int q0 = c.q0(), hq = c.head();
        if (lane == 0) {
          KB_FTR(0, g, 0);
          // order of issue = order of need: S wants K and Q, dP (issued a tile later) wants V and dO
          if (c.t == 0) {
            // K and V of an item are read by this CTA only, so they always come from DRAM: have the
            // next item's tiles brought into L2 a whole item ahead of their loads
            Cursor nx = c;
            nx.t = nx.tiles() - 1;
            cursor_next<PACKED>(a, nx, n_items, n_ktiles);
            if (nx.valid) {
#pragma unroll
              for (int p = 0; p < kPanels; ++p) {
                tma_prefetch_l2_4d(&tm_k, p * 64, nx.it.row0 + nx.it.k0, nx.it.hk, PACKED ? 0 : nx.it.b);
                tma_prefetch_l2_4d(&tm_v, p * 64, nx.it.row0 + nx.it.k0, nx.it.hk, PACKED ? 0 : nx.it.b);
              }
            }
            const int ks = n & 1;
            // the buffer held K(n - 2), then staged that item's dV / dK on their way out
            if (n >= 2) ok = mbar_wait<kRelaxedNs>(&sm.k_free[ks], ((n >> 1) - 1) & 1, ctx, kWKFree);
            if (ok) {
              mbar_expect_tx(&sm.k_full[ks], kTileBytes);
#pragma unroll
              for (int p = 0; p < kPanels; ++p)
                tma_load_4d(sm.k[ks] + p * kPanelBytes, &tm_k, &sm.k_full[ks], p * 64, c.it.row0 + c.it.k0, c.it.hk, PACKED ? 0 : c.it.b);
            }
          }
          if (ok && g >= 2) ok = mbar_wait<kRelaxedNs>(&sm.q_empty[g & 1], ((g >> 1) - 1) & 1, ctx, kWQEmpty);
          if (ok) {
            mbar_expect_tx(&sm.q_full[g & 1], kTileBytes);
#pragma unroll
            for (int p = 0; p < kPanels; ++p)
              tma_load_4d(sm.q[g & 1] + p * kPanelBytes, &tm_q, &sm.q_full[g & 1], p * 64, c.it.row0 + q0, hq, PACKED ? 0 : c.it.b);
          }
          KB_FTR(0, g, 1);
          if (ok && c.t == 0) {
            if (n >= 1) ok = mbar_wait<kRelaxedNs>(&sm.v_empty, (n - 1) & 1, ctx, kWVEmpty);
            if (ok) {
              mbar_expect_tx(&sm.v_full, kTileBytes);
#pragma unroll
              for (int p = 0; p < kPanels; ++p)
                tma_load_4d(sm.v + p * kPanelBytes, &tm_v, &sm.v_full, p * 64, c.it.row0 + c.it.k0, c.it.hk, PACKED ? 0 : c.it.b);
            }
          }
          if (ok && g >= 1) ok = mbar_wait<kRelaxedNs>(&sm.do_empty, (g - 1) & 1, ctx, kWDoEmpty);
          if (ok) {
            mbar_expect_tx(&sm.do_full, kTileBytes);
#pragma unroll
            for (int p = 0; p < kPanels; ++p)
              tma_load_4d(sm.d_o + p * kPanelBytes, &tm_do, &sm.do_full, p * 64, c.it.row0 + q0, hq, PACKED ? 0 : c.it.b);
          }
          KB_FTR(0, g, 2);
        }
      }
    } else if (warp == kStatsWarp) {
      // ------------------------------ lse / delta staging ------------------------------
      // lse and delta of the tile's query rows, two slots deep: slot g & 1 was last read while dS(g - 2) was
      // formed.  The P phase of tile g needs them the moment S(g) completes.  The loop is kept short: two 64-bit
      // multiplies per element in it cost the kernel 15 %.
      bool ok = true;
      for (Cursor c = cursor_first<PACKED>(a, n_items, n_ktiles); ok && c.valid; cursor_next<PACKED>(a, c, n_items, n_ktiles)) {
        const int g = c.g;
        const int q0 = c.q0(), hq = c.head();
        if (g >= 2) ok = mbar_wait<kRelaxedNs>(&sm.ds_ready[g & 1], ((g >> 1) - 1) & 1, ctx, kWStatsSlot);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const float* lse_row = a.lse + (c.it.b * a.lse_sb + hq * a.lse_sh) + c.it.row0 + q0 + lane;
        const float* delta_row = PACKED ? a.delta + (int64_t)hq * a.total + c.it.row0 + q0 + lane
                                        : a.delta + ((int64_t)c.it.b * a.H + hq) * T + q0 + lane;
#pragma unroll
        for (int i = 0; i < kBQ / 32; ++i) {
          const bool valid = q0 + lane + 32 * i < c.it.len;
          sm.lse_s[g & 1][lane + 32 * i] = valid ? lse_row[32 * i] : 0.f;
          sm.delta_s[g & 1][lane + 32 * i] = valid ? delta_row[32 * i] : 0.f;
        }
        mbar_arrive(&sm.stats_full[g & 1]);
      }
    } else if (warp == kMmaWarp && lane == 0) {
      // ------------------------------ MMA issuer ------------------------------
      constexpr uint32_t idesc_z = make_idesc(BF16, kBK, kBQ, false, false);  // S, dP
      constexpr uint32_t idesc_acc = make_idesc(BF16, kBK, D, false, true);   // dV, dK (A in TMEM)
      const uint32_t v_addr = smem_u32(sm.v), do_addr = smem_u32(sm.d_o);
#ifdef KB_TRACE_FUSED
      long long acc_t[12] = {0};
      long long tl = clock64();
#define KB_ACC(i) do { const long long tn_ = clock64(); acc_t[i] += tn_ - tl; tl = tn_; } while (0)
#else
#define KB_ACC(i) do { } while (0)
#endif

      // The eight instructions of a matmul are issued from rolled loops on purpose: the MMA thread shares
      // its instruction cache with compute warps that run long unrolled loops, and a short issue path
      // measured 4 % faster than the unrolled one.
      // S of tile g (item n) = K Q^T;  `new_item`: the tile opens an item, whose K has to have arrived
      auto issue_s = [&](int n, int g, bool new_item) -> bool {
        if (new_item && !mbar_wait(&sm.k_full[n & 1], (n >> 1) & 1, ctx, kWKFull)) return false;
        if (!mbar_wait(&sm.q_full[g & 1], (g >> 1) & 1, ctx, kWQFull)) return false;
        KB_ACC(9);  // waits for K, Q (counted apart from the issue of S)
        tc_fence_after();
        uint32_t k_lo = desc_lo_kmajor(smem_u32(sm.k[n & 1])), q_lo = desc_lo_kmajor(smem_u32(sm.q[g & 1]));
#pragma unroll 1
        for (int p = 0; p < D / 64; ++p, k_lo += kPanelBytes >> 4, q_lo += kPanelBytes >> 4) {
#pragma unroll
          for (int i = 0; i < 4; ++i) mma_ss_lo(tmem + kColS, k_lo + 2 * i, q_lo + 2 * i, idesc_z, p > 0 || i > 0);
        }
        mma_commit(&sm.s_ready);
        return true;
      };
      // dP of tile g (item n) = V dO^T;  `last`: the tile closes its item
      auto issue_dp = [&](int n, int g, bool new_item, bool last) -> bool {
        if (new_item && !mbar_wait(&sm.v_full, n & 1, ctx, kWVFull)) return false;
        if (!mbar_wait(&sm.do_full, g & 1, ctx, kWDoFull)) return false;
        KB_ACC(10);  // waits for V, dO (counted apart from the issue of dP)
        tc_fence_after();
        uint32_t v_lo = desc_lo_kmajor(v_addr), do_lo = desc_lo_kmajor(do_addr);
#pragma unroll 1
        for (int p = 0; p < D / 64; ++p, v_lo += kPanelBytes >> 4, do_lo += kPanelBytes >> 4) {
#pragma unroll
          for (int i = 0; i < 4; ++i) mma_ss_lo(tmem + kColDP, v_lo + 2 * i, do_lo + 2 * i, idesc_z, p > 0 || i > 0);
        }
        mma_commit(&sm.dp_ready);
        if (last) mma_commit(&sm.v_empty);  // V of this item has no reader left
        return true;
      };
      // acc += A(tmem, 16-bit at `a_col`) * B(smem tile at b_addr, MN-major)
      auto issue_acc = [&](uint32_t acc_col, uint32_t a_col, uint32_t b_addr, bool first_tile) {
        // 16 queries = 8 packed columns; queries [64 w, 64 w + 64) sit at columns 64 w ..
        uint32_t a = tmem + a_col, b_lo = desc_lo_mnmajor(b_addr, kPanelBytes);
#pragma unroll 1
        for (int p = 0; p < kBQ / 64; ++p, a += 64, b_lo += 4 * (2048 >> 4)) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            mma_ts_lo(tmem + acc_col, a + 8 * i, b_lo + i * (2048 >> 4), idesc_acc, !first_tile || p > 0 || i > 0);
        }
      };
      // This thread keeps no cursor: all it needs of the schedule is how many tiles each live item has.
      // Tiles of the first live item at or after `item` (stride gridDim.x), 0 if there is none.
      auto next_live = [&](int& item) -> int {
        Item prev;
        prev.b = -1;
        for (; item < n_items; item += gridDim.x) {
          const Item it = decode_item<PACKED>(a, item, n_ktiles, prev);
          if (it.qr.begin < it.qr.end) return (it.qr.end - it.qr.begin) * a.group;
        }
        return 0;
      };

      int item = blockIdx.x;
      int cnt = next_live(item);  // tiles of the current item
      int n = 0, g = 0;           // live items, tiles so far
      bool ok = cnt > 0 && issue_s(0, 0, true) && issue_dp(0, 0, true, cnt == 1);
      KB_ACC(11);
      if constexpr (MID) {
        int cnt_next = 0, t = 0;
        // One tile: dV(g), S(g+1), dK(g), dP(g+1), with whether the tile opens / closes its item known at compile
        // time (inside an item: no tests of either, constant accumulate flags, no item bookkeeping; every scalar
        // instruction between two MMAs of this thread is time the chain P -> dV -> S waits).
        auto tile = [&](auto first_c, auto last_c) -> bool {
          constexpr bool first = decltype(first_c)::value, last = decltype(last_c)::value;
          KB_FTR(1, g, 0);
          KB_ACC(0);  // loop
          // dV(g) += P(g) dO(g)
          if (!mbar_wait(&sm.p_ready, g & 1, ctx, kWPReady)) return false;
          KB_ACC(1);  // wait p_ready
          // the first MMAs of an item overwrite dV / dK: the epilogue warps must have read the old ones
          if (first && n > 0 && !mbar_wait(&sm.dv_free, (n - 1) & 1, ctx, kWAccFree)) return false;
          KB_FTR(1, g, 1);
          KB_ACC(2);  // wait dv_free
          tc_fence_after();
          issue_acc(kColDV, kColS, do_addr, first);
          mma_commit(&sm.do_empty);
          if (last) mma_commit(&sm.dv_done);  // the epilogue warps start on dV while dK(last) still runs
          KB_FTR(1, g, 2);
          KB_ACC(3);  // issue dV
          // S(g+1): of this item, or the first of the next live one.  (Looking for the next item before the wait for
          // P instead, off the chain, as the other classes' loop below does, measured 1 % slower in this one.)
          if (last) {
            item += gridDim.x;
            cnt_next = next_live(item);
          }
          const bool more = !last || cnt_next > 0;
          if (more && !issue_s(last ? n + 1 : n, g + 1, last)) return false;
          KB_FTR(1, g, 3);
          KB_ACC(4);  // S(g+1) incl. the look for the next item
          // dK(g) += dS(g) Q(g)
          if (!mbar_wait(&sm.ds_ready[g & 1], (g >> 1) & 1, ctx, kWDsReady)) return false;
          KB_ACC(5);  // wait ds_ready
          if (first && n > 0 && !mbar_wait(&sm.dk_free, (n - 1) & 1, ctx, kWAccFree)) return false;
          KB_ACC(6);  // wait dk_free
          KB_FTR(1, g, 4);
          tc_fence_after();
          issue_acc(kColDK, kColDP, smem_u32(sm.q[g & 1]), first);
          mma_commit(&sm.q_empty[g & 1]);
          if (last) mma_commit(&sm.dk_done);
          KB_FTR(1, g, 5);
          KB_ACC(7);  // issue dK
          // dP(g+1)
          if (more && !issue_dp(last ? n + 1 : n, g + 1, last, last ? cnt_next == 1 : t + 1 == cnt - 1)) return false;
          KB_ACC(8);  // dP(g+1)
          return true;
        };
        while (ok) {
          cnt_next = 0;
          for (t = 0; ok && t < cnt; ++t, ++g) {
            const bool first = t == 0, last = t == cnt - 1;
            using Yes = std::true_type;
            using No = std::false_type;
            if (!first && !last) ok = tile(No{}, No{});
            else if (first && !last) ok = tile(Yes{}, No{});
            else if (!first) ok = tile(No{}, Yes{});
            else ok = tile(Yes{}, Yes{});
          }
          if (!ok || cnt_next == 0) break;
          cnt = cnt_next;
          ++n;
        }
      } else {
        // (the same sequence written out in the loop: through the lambda above these classes measured 1 % slower)
        while (ok) {
          int cnt_next = 0;
          for (int t = 0; ok && t < cnt; ++t, ++g) {
            const bool first = t == 0, last = t == cnt - 1;
            // The look for the next live item (a decode per candidate) is done here, before the wait for P: from
            // that wait to the issue of S(g+1) the thread is on the kernel's critical chain.
            if (last) {
              item += gridDim.x;
              cnt_next = next_live(item);
            }
            const bool more = !last || cnt_next > 0;
            const int n_next = last ? n + 1 : n;                           // item of tile g + 1
            const bool dp_last = last ? cnt_next == 1 : t + 1 == cnt - 1;  // tile g + 1 closes its item
            KB_FTR(1, g, 0);
            KB_ACC(0);  // loop
            // dV(g) += P(g) dO(g)
            if (!mbar_wait(&sm.p_ready, g & 1, ctx, kWPReady)) { ok = false; break; }
            KB_ACC(1);  // wait p_ready
            // the first MMAs of an item overwrite dV / dK: the epilogue warps must have read the old ones
            if (first && n > 0 && !mbar_wait(&sm.dv_free, (n - 1) & 1, ctx, kWAccFree)) { ok = false; break; }
            KB_FTR(1, g, 1);
            KB_ACC(2);  // wait dv_free
            tc_fence_after();
            issue_acc(kColDV, kColS, do_addr, first);
            mma_commit(&sm.do_empty);
            if (last) mma_commit(&sm.dv_done);  // the epilogue warps start on dV while dK(last) still runs
            KB_FTR(1, g, 2);
            KB_ACC(3);  // issue dV
            // S(g+1): of this item, or the first of the next live one
            if (more && !issue_s(n_next, g + 1, last)) { ok = false; break; }
            KB_FTR(1, g, 3);
            KB_ACC(4);  // S(g+1) incl. the look for the next item
            // dK(g) += dS(g) Q(g)
            if (!mbar_wait(&sm.ds_ready[g & 1], (g >> 1) & 1, ctx, kWDsReady)) { ok = false; break; }
            KB_ACC(5);  // wait ds_ready
            if (first && n > 0 && !mbar_wait(&sm.dk_free, (n - 1) & 1, ctx, kWAccFree)) { ok = false; break; }
            KB_ACC(6);  // wait dk_free
            KB_FTR(1, g, 4);
            tc_fence_after();
            issue_acc(kColDK, kColDP, smem_u32(sm.q[g & 1]), first);
            mma_commit(&sm.q_empty[g & 1]);
            if (last) mma_commit(&sm.dk_done);
            KB_FTR(1, g, 5);
            KB_ACC(7);  // issue dK
            // dP(g+1)
            if (more && !issue_dp(n_next, g + 1, last, dp_last)) { ok = false; break; }
            KB_ACC(8);  // dP(g+1)
          }
          if (cnt_next == 0) break;
          cnt = cnt_next;
          ++n;
        }
      }
#ifdef KB_TRACE_FUSED
      if (blockIdx.x == 60)
        for (int i = 0; i < 12; ++i) g_ftrace[3][62][i % 8 + 0] = 0, g_ftrace[3][60 + i / 8][i % 8] = acc_t[i];
#endif
    } else if (warp == kSpillWarp && lane == 0) {
      // ------------------------------ dS tiles to the scratch buffer ------------------------------
      for (Cursor c = cursor_first<PACKED>(a, n_items, n_ktiles); c.valid; cursor_next<PACKED>(a, c, n_items, n_ktiles)) {
        if (!mbar_wait<kRelaxedNs>(&sm.ds_ready[c.g & 1], (c.g >> 1) & 1, ctx, kWSpill)) break;
        bulk_store(ds_slot<PACKED>(a, c.it.b, c.it.row0, c.head(), c.it.kt, n_ktiles, c.tq), sm.ds, kDsTileBytes);
        tma_store_commit();
        tma_store_wait_read();
        mbar_arrive(&sm.ds_free);  // the compute warps may form the next dS in the buffer
      }
      tma_store_wait_all();
    }
  }
  else if (warp < kEpiWarp0) {
    // ------------------------------ compute warps ------------------------------
    setmaxnreg_inc<kRegsCompute>();
    const int row = (warp & 3) * 32 + lane;
    const int half = warp >> 2;  // which 64 query columns of each tile this warpgroup owns
    const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t t_s = t_lane + kColS + half * 64, t_dp = t_lane + kColDP + half * 64;
    uint8_t* ds_row = sm.ds + half * kPanelBytes + row * 128;
    const float scale = a.scale_log2;
    int lo = 0, hi = 0;  // live query columns of this key row: [lo, hi)
    bool ok = true;
    for (Cursor c = cursor_first<PACKED>(a, n_items, n_ktiles); ok && c.valid; cursor_next<PACKED>(a, c, n_items, n_ktiles)) {
      const int g = c.g;
      if (c.t == 0) {
        const int xi = c.it.k0 + row;
        lo = hi = 0;
        if (xi < c.it.len) {
          const int xc = kb_fastdiv(xi, a.fd_c);
          lo = xc * a.c;
          const int64_t h64 = (int64_t)(xc + a.back + 1) * a.c;
          hi = h64 < c.it.len ? (int)h64 : c.it.len;
        }
      }
      const int y0 = c.q0() + half * 64;  // first query column this thread handles
      const float* lse_c = sm.lse_s[g & 1] + half * 64;
      const float* delta_c = sm.delta_s[g & 1] + half * 64;

      // ---- phase 1: P = 2^(S * scale - lse) for this thread's 64 columns, 16-bit, back into TMEM
      if (threadIdx.x == 0) KB_FTR(2, g, 0);
      ok = __all_sync(0xffffffffu, mbar_wait(&sm.s_ready, g & 1, ctx, kWSReady));
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&sm.stats_full[g & 1], (g >> 1) & 1, ctx, kWStatsFull));
      if (!ok) break;
      tc_fence_after();
      if (threadIdx.x == 0) KB_FTR(2, g, 1);
      const bool warp_full = __all_sync(0xffffffffu, lo <= y0 && y0 + 64 <= hi);
      float p[64];
      {
        uint32_t s[64];
        tmem_ld32(t_s, reinterpret_cast<uint32_t(&)[32]>(s[0]));
        tmem_ld32(t_s + 32, reinterpret_cast<uint32_t(&)[32]>(s[32]));
        tmem_wait_ld();
        // 32 columns at a time, with warp-wide votes when the block is not live throughout: a group that
        // is masked for every row of the warp needs no exponentials, one that is live for every row no
        // selects (chunk boundaries that are multiples of 32 never leave a mixed group)
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c0 = y0 + cc * 32;
          const bool all_dead = !warp_full && __all_sync(0xffffffffu, c0 + 32 <= lo || c0 >= hi);
          if (all_dead) {
#pragma unroll
            for (int i = 0; i < 32; ++i) p[cc * 32 + i] = 0.f;
            continue;
          }
#pragma unroll
          for (int i = cc * 32; i < cc * 32 + 32; i += 4) {
            const float4 lv = *reinterpret_cast<const float4*>(lse_c + i);
            p[i + 0] = ex2_approx(fmaf(__uint_as_float(s[i + 0]), scale, -lv.x));
            p[i + 1] = ex2_approx(fmaf(__uint_as_float(s[i + 1]), scale, -lv.y));
            p[i + 2] = ex2_approx(fmaf(__uint_as_float(s[i + 2]), scale, -lv.z));
            p[i + 3] = ex2_approx(fmaf(__uint_as_float(s[i + 3]), scale, -lv.w));
          }
          if (!warp_full && !__all_sync(0xffffffffu, lo <= c0 && c0 + 32 <= hi)) {
#pragma unroll
            for (int i = cc * 32; i < cc * 32 + 32; ++i) p[i] = (y0 + i >= lo && y0 + i < hi) ? p[i] : 0.f;
          }
        }
      }
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

      // ---- phase 2: dS = P * (dP - delta), 16-bit: over dP in TMEM (operand of dK) and into shared
      // memory (row = key, 64 queries = one 128-byte row of the thread's panel) for the scratch copy
      if (threadIdx.x == 0) KB_FTR(2, g, 2);
      ok = __all_sync(0xffffffffu, mbar_wait(&sm.dp_ready, g & 1, ctx, kWDpReady));
      if (!ok) break;
      if (threadIdx.x == 0) KB_FTR(2, g, 3);
      tc_fence_after();
      uint32_t ds[32];
      {
        uint32_t dp[64];
        tmem_ld32(t_dp, reinterpret_cast<uint32_t(&)[32]>(dp[0]));
        tmem_ld32(t_dp + 32, reinterpret_cast<uint32_t(&)[32]>(dp[32]));
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float4 dv = *reinterpret_cast<const float4*>(delta_c + 2 * i);
          const int e = 2 * i;
          ds[i] = pack16x2<BF16>(p[e] * (__uint_as_float(dp[e]) - dv.x), p[e + 1] * (__uint_as_float(dp[e + 1]) - dv.y));
          ds[i + 1] = pack16x2<BF16>(p[e + 2] * (__uint_as_float(dp[e + 2]) - dv.z), p[e + 3] * (__uint_as_float(dp[e + 3]) - dv.w));
        }
      }
      tmem_st16(t_dp, reinterpret_cast<const uint32_t(&)[16]>(ds[0]));
      tmem_st16(t_dp + 16, reinterpret_cast<const uint32_t(&)[16]>(ds[16]));
      // the bulk copy that carries dS(g - 1) to the scratch buffer must have read it
      if (g > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(&sm.ds_free, (g - 1) & 1, ctx, kWDsFree));
        if (!ok) break;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(ds_row + ((j ^ (row & 7)) << 4)) = make_uint4(ds[4 * j], ds[4 * j + 1], ds[4 * j + 2], ds[4 * j + 3]);
      fence_proxy_async();  // the bulk copy reads shared memory through the async proxy
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&sm.ds_ready[g & 1]);
      if (threadIdx.x == 0) KB_FTR(2, g, 4);
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    // End of an item: dV and dK (the latter carries the softmax scale) go TMEM -> 16-bit -> shared
    // memory (the item's own K buffer, whose last reader was the item's last S) -> TMA store.
    setmaxnreg_dec<kRegsEpi>();
    const int row = (warp & 3) * 32 + lane;
    const int etid = threadIdx.x - kEpiWarp0 * 32;
    const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    int n = 0;
    bool ok = true;
    Item it;
    it.b = -1;
    for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
      it = decode_item<PACKED>(a, item, n_ktiles, it);
      const int kr = it.k0 + row;
      if (it.qr.begin >= it.qr.end) {
        // the whole key tile lies in the padding: its gradients are zeros (rare; plain stores).  A packed
        // batch has no padding rows: a tile past the sequence's end owns nothing.
        if (!PACKED && kr < T) {
          const int64_t off = it.b * a.dkv_sb + it.hk * a.dkv_sh + kr * a.dkv_st;  // one head per key/value head
          uint4* dv_row = reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.dv) + off);
          uint4* dk_row = reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.dk) + off);
#pragma unroll
          for (int i = 0; i < D * 2 / 16; ++i) {
            dv_row[i] = make_uint4(0, 0, 0, 0);
            dk_row[i] = make_uint4(0, 0, 0, 0);
          }
        }
        continue;
      }
      uint8_t* stage = sm.k[n & 1];
      // Packed batch, last key tile of a sequence: the rows below it belong to the next sequence, so the tile
      // cannot leave as a box store; every thread writes its own row (one such tile per sequence and head).
      const bool partial = PACKED && it.k0 + kBK > it.len;
      const int64_t row_off = it.hk * a.dkv_sh + (int64_t)(it.row0 + kr) * a.dkv_st;  // used by the partial tile only
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const float mul = which ? a.sm_scale : 1.f;
        // dV is complete after the item's last dV MMA (every S that reads the K buffer ran before it),
        // dK one matmul later.  All four warps must take the same exit: they meet at named barriers.
        ok = named_barrier_and(1, kEpiThreads, mbar_wait<kRelaxedNs>(which ? &sm.dk_done : &sm.dv_done, n & 1, ctx, kWAccDone));
        if (!ok) break;
        if (etid == 0) KB_FTR(3, n, which);
        tc_fence_after();
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t r[32];
          tmem_ld32(t_lane + (which ? kColDK : kColDV) + cc * 32, r);
          tmem_wait_ld();
          if (cc == D / 32 - 1) {
            tc_fence_before();
            mbar_arrive(which ? &sm.dk_free : &sm.dv_free);  // the next item may overwrite this accumulator
          }
          uint8_t* prow = stage + (cc / 2) * kPanelBytes + row * 128;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 w;
            w.x = pack16x2<BF16>(__uint_as_float(r[8 * q4 + 0]) * mul, __uint_as_float(r[8 * q4 + 1]) * mul);
            w.y = pack16x2<BF16>(__uint_as_float(r[8 * q4 + 2]) * mul, __uint_as_float(r[8 * q4 + 3]) * mul);
            w.z = pack16x2<BF16>(__uint_as_float(r[8 * q4 + 4]) * mul, __uint_as_float(r[8 * q4 + 5]) * mul);
            w.w = pack16x2<BF16>(__uint_as_float(r[8 * q4 + 6]) * mul, __uint_as_float(r[8 * q4 + 7]) * mul);
            const int chunk = (cc & 1) * 4 + q4;  // 16-byte chunk within the 128-byte panel row
            if (partial) {
              if (kr < it.len)
                reinterpret_cast<uint4*>(static_cast<uint16_t*>(which ? a.dk : a.dv) + row_off)[cc * 4 + q4] = w;
            } else {
              *reinterpret_cast<uint4*>(prow + ((chunk ^ (row & 7)) << 4)) = w;
            }
          }
        }
        fence_proxy_async();
        named_barrier_sync(1, kEpiThreads);
        if (etid == 0) {
          if (!partial) {
#pragma unroll
            for (int p = 0; p < kPanels; ++p)
              tma_store_4d(which ? &tm_dk : &tm_dv, stage + p * kPanelBytes, p * 64, it.row0 + it.k0, it.hk, PACKED ? 0 : it.b);
            tma_store_commit();
            tma_store_wait_read();
          }
          if (which == 1) mbar_arrive(&sm.k_free[n & 1]);  // K(n + 2) may land in the buffer
        }
        named_barrier_sync(1, kEpiThreads);  // `stage` may be overwritten
      }
      if (!ok) break;
      ++n;
    }
    if (etid == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
#ifdef KB_TRACE_FUSED
  if (threadIdx.x == 0 && blockIdx.x == 60) {
    g_ftrace[3][63][2] = clock64();
    g_ftrace[3][63][3] = (long long)globaltimer_ns();
  }
#endif
  if (warp == kMmaWarp) {
    if (sm.abort_flag) __nanosleep(1000000);  // let copies still in flight land before the CTA goes away
    tmem_dealloc(tmem, kTmemCols);
  }
}

// ---- delta = rowsum(O * dO), one CTA per 128 rows (kernel.py:453-514) ----
struct DeltaArgs {
  const uint16_t* o;
  const uint16_t* d_o;
  int64_t o_sb, o_sh, o_st, do_sb, do_sh, do_st;
  float* delta;
  const int32_t* lens;
  int64_t lens_stride;
  int32_t H, T;
  const int32_t* cu;  // packed batch (see FusedArgs): rows of sequence b start at cu[b], delta is [H, total]
  int32_t total;
};

template <int D, bool BF16>
__global__ void __launch_bounds__(256) sa_bwd_delta_kernel(const DeltaArgs a) {
  const int b = blockIdx.z, h = blockIdx.y, x0 = blockIdx.x * kBQ;
  const int T = a.T;
  int len = a.lens ? kb_clamp_len(a.lens[(int64_t)b * a.lens_stride], T) : T;
  int row0 = 0;
  if (a.cu) {
    row0 = a.cu[b];
    len = kb_min_i32(a.cu[b + 1] - row0, T);
    if (x0 >= len) return;  // a packed batch has no padding rows to clear
  }
  // rows a CTA may write: the tensor's in the padded layout (rows past len get 0), the sequence's when packed
  const int row_end = a.cu ? len : T;
  float* delta_out = a.cu ? a.delta + (int64_t)h * a.total + row0 : a.delta + ((int64_t)b * a.H + h) * T;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // a group of D/8 lanes reads one row as 16-byte chunks; warp w covers rows 16 w .. 16 w + 15
  constexpr int kLanesPerRow = D / 8, kRowsPerIter = 32 / kLanesPerRow, kIters = 16 / kRowsPerIter;
  const int sub = lane / kLanesPerRow, chunk = lane % kLanesPerRow;
  const uint16_t* o_base = a.o + b * a.o_sb + h * a.o_sh + (int64_t)row0 * a.o_st;
  const uint16_t* g_base = a.d_o + b * a.do_sb + h * a.do_sh + (int64_t)row0 * a.do_st;
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
    const int r = x0 + 16 * warp + it * kRowsPerIter + sub;
    if (chunk == 0 && r < row_end) delta_out[r] = part;
  }
}

// ---- dQ = sm_scale * sum_j dS_j^T K_j over the saved dS tiles ----
// Persistent, one CTA per SM, six warps: warps 0-3 epilogue (thread = query row = TMEM lane),
// warp 4 producer (one lane: a 32 KB bulk copy of dS and a TMA tile of K per stage, three stages),
// warp 5 MMA issuer (one lane) and TMEM owner.  The accumulator is double buffered in TMEM so that
// the MMAs of the next item run while the epilogue warps convert and store the finished one.
constexpr int kDqStages = tiles::kDqStages;
constexpr int kDqThreads = 192;
constexpr int kDqProducerWarp = 4, kDqMmaWarp = 5;
constexpr uint32_t kDqTmemCols = 256;

template <int D>
struct alignas(1024) DqSmem {
  uint8_t ds[kDqStages][kDsTileBytes];
  uint8_t k[kDqStages][kBK * D * 2];
  uint8_t out[kBQ * D * 2];
  uint64_t full[kDqStages], empty[kDqStages], acc_done[2], acc_free[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct DqItem {
  int b, h, qt, len;
  int row0;        // first row of the sequence in the tensor maps (packed batch: cu[b]; else 0)
  KbTileRange kr;  // key tiles [begin, end) the query tile visits: the forward schedule
};
template <bool PACKED>
__device__ __forceinline__ DqItem decode_dq_item(const FusedArgs& a, int item, int n_qtiles, const DqItem& prev) {
  DqItem it;
  const int bh = kb_fastdiv(item, a.fd_tiles);
  it.qt = item - bh * n_qtiles;
  it.b = kb_fastdiv(bh, a.fd_H);
  it.h = bh - it.b * a.H;
  it.row0 = 0;
  if (PACKED) {
    if (it.b == prev.b) {
      it.row0 = prev.row0;
      it.len = prev.len;
    } else {
      it.row0 = a.cu[it.b];
      it.len = kb_min_i32(a.cu[it.b + 1] - it.row0, a.T);
    }
  } else {
    it.len = !a.lens ? a.T : (it.b == prev.b ? prev.len : kb_clamp_len(a.lens[(int64_t)it.b * a.lens_stride], a.T));
  }
  it.kr = kb_fwd_kv_range_fd(it.qt * kBQ, kBQ, kBK, it.len, a.c, a.back, a.fd_c);
  return it;
}

template <int D, bool BF16, bool PACKED>
__global__ void __launch_bounds__(kDqThreads, 1)
sa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_dq, const FusedArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  DqSmem<D>& sm = *reinterpret_cast<DqSmem<D>*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T = a.T;
  const int n_tiles_t = kb_cdiv_i32(T, kBQ);  // query tiles = key tiles per sequence
  const int n_items = a.B * a.H * n_tiles_t;

  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0 && a.status) {
      atomicExch(a.status, KB_ERR_DEVICE_TIMEOUT);
      atomicExch(a.status + 1, kErrSmemAlign);
    }
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kDqStages; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.acc_done[i], 1);
      mbar_init(&sm.acc_free[i], 128);
    }
    sm.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kDqMmaWarp) tmem_alloc(&sm.tmem_base, kDqTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const WaitCtx ctx{&sm.abort_flag, a.status};
  constexpr int kPanels = D / 64;
  constexpr uint32_t kTileBytes = 128 * D * 2;

  // u counts the (query tile, key tile) pairs of this CTA so far, m its items with at least one pair
  if (warp == kDqProducerWarp) {
    if (lane == 0) {
      prefetch_tensormap(&tm_k);
      int u = 0;
      bool ok = true;
      DqItem it;
      it.b = -1;
      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
        it = decode_dq_item<PACKED>(a, item, n_tiles_t, it);
        for (int j = it.kr.begin; j < it.kr.end; ++j, ++u) {
          const int s = u % kDqStages;
          if (u >= kDqStages && !mbar_wait<kRelaxedNs>(&sm.empty[s], ((u / kDqStages) - 1) & 1, ctx, kWDqEmpty)) { ok = false; break; }
          // the slot this query tile has in key tile j's list: both schedules name the same pairs
          const KbTileRange qr = kb_bwd_q_range_fd(j * kBK, kBQ, kBK, it.len, a.c, a.back, a.fd_c);
          mbar_expect_tx(&sm.full[s], kDsTileBytes + kTileBytes);
          bulk_load(sm.ds[s], ds_slot<PACKED>(a, it.b, it.row0, it.h, j, n_tiles_t, it.qt - qr.begin), kDsTileBytes, &sm.full[s]);
#pragma unroll
          for (int p = 0; p < kPanels; ++p)
            tma_load_4d(sm.k[s] + p * kPanelBytes, &tm_k, &sm.full[s], p * 64, it.row0 + j * kBK, kb_fastdiv(it.h, a.fd_group), PACKED ? 0 : it.b);
        }
      }
    }
  } else if (warp == kDqMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BF16, kBQ, D, true, true);  // A = dS read MN-major (rows = keys), B = K MN-major
      int u = 0, m = 0;
      bool ok = true;
      DqItem it;
      it.b = -1;
      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
        it = decode_dq_item<PACKED>(a, item, n_tiles_t, it);
        if (it.kr.begin >= it.kr.end) continue;
        const uint32_t acc = tmem + (m & 1) * 128;
        if (m >= 2 && !mbar_wait(&sm.acc_free[m & 1], ((m >> 1) - 1) & 1, ctx, kWDqAccFree)) break;
        for (int j = it.kr.begin; j < it.kr.end; ++j, ++u) {
          const int s = u % kDqStages;
          if (!mbar_wait(&sm.full[s], (u / kDqStages) & 1, ctx, kWDqFull)) { ok = false; break; }
          tc_fence_after();
          uint32_t ds_lo = desc_lo_mnmajor(smem_u32(sm.ds[s]), kPanelBytes), k_lo = desc_lo_mnmajor(smem_u32(sm.k[s]), kPanelBytes);
#pragma unroll 1
          for (int h = 0; h < kBK / 64; ++h, ds_lo += 4 * (2048 >> 4), k_lo += 4 * (2048 >> 4)) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              mma_ss_lo(acc, ds_lo + i * (2048 >> 4), k_lo + i * (2048 >> 4), idesc, j > it.kr.begin || h > 0 || i > 0);
          }
          mma_commit(&sm.empty[s]);
        }
        if (ok) mma_commit(&sm.acc_done[m & 1]);
        ++m;
      }
    }
  } else {
    const int row = warp * 32 + lane;
    const uint32_t t_lane = tmem + ((uint32_t)(warp * 32) << 16);
    int m = 0;
    bool ok = true;
    DqItem it;
    it.b = -1;
    for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
      it = decode_dq_item<PACKED>(a, item, n_tiles_t, it);
      const int qi = it.qt * kBQ + row;
      if (it.kr.begin >= it.kr.end) {
        // the whole query tile lies in the padding: its gradient is zero (rare; plain stores); a packed batch
        // has no padding rows
        if (!PACKED && qi < T) {
          uint4* dq_row = reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.dq) + it.b * a.dq_sb + it.h * a.dq_sh + qi * a.dq_st);
#pragma unroll
          for (int i = 0; i < D * 2 / 16; ++i) dq_row[i] = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      // packed batch, last query tile of a sequence: the rows below belong to the next sequence, so no box
      // store; every thread writes its own row
      const bool partial = PACKED && it.qt * kBQ + kBQ > it.len;
      // all four warps must take the same exit: they meet at named barriers below
      ok = named_barrier_and(1, 128, mbar_wait<kRelaxedNs>(&sm.acc_done[m & 1], (m >> 1) & 1, ctx, kWDqAccDone));
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t r[32];
        tmem_ld32(t_lane + (m & 1) * 128 + cc * 32, r);
        tmem_wait_ld();
        if (cc == D / 32 - 1) {
          tc_fence_before();
          mbar_arrive(&sm.acc_free[m & 1]);
        }
        uint8_t* prow = sm.out + (cc / 2) * kPanelBytes + row * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 w;
          w.x = pack16x2<BF16>(__uint_as_float(r[8 * q4 + 0]) * a.sm_scale, __uint_as_float(r[8 * q4 + 1]) * a.sm_scale);
          w.y = pack16x2<BF16>(__uint_as_float(r[8 * q4 + 2]) * a.sm_scale, __uint_as_float(r[8 * q4 + 3]) * a.sm_scale);
          w.z = pack16x2<BF16>(__uint_as_float(r[8 * q4 + 4]) * a.sm_scale, __uint_as_float(r[8 * q4 + 5]) * a.sm_scale);
          w.w = pack16x2<BF16>(__uint_as_float(r[8 * q4 + 6]) * a.sm_scale, __uint_as_float(r[8 * q4 + 7]) * a.sm_scale);
          const int chunk = (cc & 1) * 4 + q4;
          if (partial) {
            if (qi < it.len)
              reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.dq) + it.h * a.dq_sh + (int64_t)(it.row0 + qi) * a.dq_st)[cc * 4 + q4] = w;
          } else {
            *reinterpret_cast<uint4*>(prow + ((chunk ^ (row & 7)) << 4)) = w;
          }
        }
      }
      fence_proxy_async();
      named_barrier_sync(1, 128);
      if (threadIdx.x == 0 && !partial) {
#pragma unroll
        for (int p = 0; p < kPanels; ++p)
          tma_store_4d(&tm_dq, sm.out + p * kPanelBytes, p * 64, it.row0 + it.qt * kBQ, it.h, PACKED ? 0 : it.b);
        tma_store_commit();
        tma_store_wait_read();
      }
      named_barrier_sync(1, 128);  // the staging tile may be overwritten
      ++m;
    }
    if (threadIdx.x == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kDqMmaWarp) {
    if (sm.abort_flag) __nanosleep(1000000);
    tmem_dealloc(tmem, kDqTmemCols);
  }
}

template <int D, bool BF16, bool PACKED>
int launch_fused(const kb_sa_bwd_params& p, int32_t c, int32_t back, cudaStream_t s) {
  CUtensorMap tm_k, tm_v, tm_q, tm_do, tm_dk, tm_dv, tm_dq;
  const int32_t Hk = p.H_kv > 0 ? p.H_kv : p.H;
  // a packed batch is ONE batch entry of `total_rows` rows as far as the maps go
  const int32_t mB = PACKED ? 1 : p.B, mT = PACKED ? p.total_rows : p.T;
  if (!make_tile_map_4d(&tm_k, p.k, mB, Hk, mT, D, kBK) || !make_tile_map_4d(&tm_v, p.v, mB, Hk, mT, D, kBK) ||
      !make_tile_map_4d(&tm_q, p.q, mB, p.H, mT, D, kBQ) || !make_tile_map_4d(&tm_do, p.d_o, mB, p.H, mT, D, kBQ) ||
      !make_tile_map_4d(&tm_dk, out_view(p.dk, p.dkv_stride, Hk, mT, D), mB, Hk, mT, D, kBK) ||
      !make_tile_map_4d(&tm_dv, out_view(p.dv, p.dkv_stride, Hk, mT, D), mB, Hk, mT, D, kBK) ||
      !make_tile_map_4d(&tm_dq, out_view(p.dq, p.dq_stride, p.H, mT, D), mB, p.H, mT, D, kBQ))
    return KB_ERR_UNSUPPORTED;
  const int n_tiles = kb_cdiv_i32(p.T, kBQ);
  const int64_t n_items = (int64_t)p.B * p.H * n_tiles;
  if (n_items > (int64_t)1 << 30) return KB_ERR_TOO_LARGE;
  int dev = 0, n_sm = 0;
  if (!device_sm_count(&dev, &n_sm)) return KB_ERR_LAUNCH;
  const unsigned grid = (unsigned)(n_items < n_sm ? n_items : n_sm);  // persistent: one CTA per SM (dQ kernel)
  const int64_t n_items_main = (int64_t)p.B * Hk * n_tiles;
  const unsigned grid_main = (unsigned)(n_items_main < n_sm ? n_items_main : n_sm);

  // the class of long items of fully live tiles gets the main kernel with the second copy of the issue sequence
  const bool mid = D == 128 && c >= 128;
  auto main_kern = mid ? sa_bwd_fused_kernel<D, BF16, PACKED, D == 128> : sa_bwd_fused_kernel<D, BF16, PACKED, false>;
  auto dq_kern = sa_bwd_dq_kernel<D, BF16, PACKED>;
  static_assert(sizeof(FusedSmem<D>) <= 232448 && sizeof(DqSmem<D>) <= 232448, "shared memory exceeds the 227 KB a CTA may have");
  static std::atomic<bool> main_opted_in[kMaxDevices], dq_opted_in[kMaxDevices];
  static std::atomic<bool> main_mid_opted_in[kMaxDevices];
  KB_CUDA_TRY(opt_in_smem_once(main_kern, sizeof(FusedSmem<D>), dev, mid ? main_mid_opted_in : main_opted_in));
  KB_CUDA_TRY(opt_in_smem_once(dq_kern, sizeof(DqSmem<D>), dev, dq_opted_in));

  DeltaArgs da;
  da.o = static_cast<const uint16_t*>(p.o.data);
  da.d_o = static_cast<const uint16_t*>(p.d_o.data);
  da.o_sb = p.o.stride[0];
  da.o_sh = p.o.stride[1];
  da.o_st = p.o.stride[2];
  da.do_sb = p.d_o.stride[0];
  da.do_sh = p.d_o.stride[1];
  da.do_st = p.d_o.stride[2];
  da.delta = p.delta_ws;
  da.lens = p.lens;
  da.lens_stride = p.lens_stride;
  da.H = p.H;
  da.T = p.T;
  da.cu = PACKED ? p.cu_seqlens : nullptr;
  da.total = PACKED ? p.total_rows : 0;
  if (PACKED) da.o_sb = da.do_sb = 0;  // the sequence's first row carries the batch offset
  if (!(p.flags & KB_FLAG_BWD_SKIP_DELTA)) {
    sa_bwd_delta_kernel<D, BF16><<<dim3(n_tiles, p.H, p.B), 256, 0, s>>>(da);
    KB_LAUNCH_CHECK("sa_bwd_delta_kernel");
  }

  FusedArgs fa;
  fa.lse = p.lse;
  {
    const kb_tensor4 qv = out_view(p.dq, p.dq_stride, p.H, mT, D), kv = out_view(p.dk, p.dkv_stride, Hk, mT, D);
    fa.dq_sb = qv.stride[0], fa.dq_sh = qv.stride[1], fa.dq_st = qv.stride[2];
    fa.dkv_sb = kv.stride[0], fa.dkv_sh = kv.stride[1], fa.dkv_st = kv.stride[2];
    const bool lse_packed = p.lse_stride[0] == 0 && p.lse_stride[1] == 0;
    fa.lse_sb = lse_packed ? (int64_t)p.H * mT : p.lse_stride[0];
    fa.lse_sh = lse_packed ? (int64_t)mT : p.lse_stride[1];
    if (PACKED) fa.dq_sb = fa.dkv_sb = fa.lse_sb = 0;
  }
  fa.cu = PACKED ? p.cu_seqlens : nullptr;
  fa.total = PACKED ? p.total_rows : 0;
  fa.n_ptiles = PACKED ? packed_tiles(p.total_rows, p.B) : 0;
  fa.delta = p.delta_ws;
  fa.ds_ws = static_cast<uint8_t*>(p.ds_ws);
  fa.dk = p.dk;
  fa.dv = p.dv;
  fa.dq = p.dq;
  fa.lens = p.lens;
  fa.lens_stride = p.lens_stride;
  fa.B = p.B;
  fa.H = p.H;
  fa.T = p.T;
  fa.c = c;
  fa.back = back;
  fa.W = fused_slots(p.T, c, back);
  fa.fd_tiles = kb_fastdiv_make(n_tiles);
  fa.Hk = Hk;
  fa.group = p.H / Hk;
  fa.fd_H = kb_fastdiv_make(p.H);
  fa.fd_Hk = kb_fastdiv_make(Hk);
  fa.fd_group = kb_fastdiv_make(p.H / Hk);
  fa.fd_c = kb_fastdiv_make(c);
  fa.scale_log2 = p.sm_scale * kLog2e;
  fa.sm_scale = p.sm_scale;
  fa.status = p.status;
  if (!(p.flags & KB_FLAG_BWD_SKIP_DKDV)) {
    main_kern<<<grid_main, kThreads, sizeof(FusedSmem<D>), s>>>(tm_k, tm_v, tm_q, tm_do, tm_dk, tm_dv, fa);
    KB_LAUNCH_CHECK("sa_bwd_fused_kernel");
  }
  if (!(p.flags & KB_FLAG_BWD_SKIP_DQ)) {
    dq_kern<<<grid, kDqThreads, sizeof(DqSmem<D>), s>>>(tm_k, tm_dq, fa);
    KB_LAUNCH_CHECK("sa_bwd_dq_kernel");
  }
  return KB_OK;
}

}  // namespace

#ifdef KB_TRACE_FUSED
}  // namespace kb
extern "C" __attribute__((visibility("default"))) int kb_debug_trace_fused(long long* out) {
  return (int)cudaMemcpyFromSymbol(out, kb::g_ftrace, sizeof(kb::g_ftrace));
}
namespace kb {
#endif

// Bytes of dS scratch the single-evaluation backward needs; c and back already clamped to T.
size_t sa_bwd_fused_workspace_bytes(int32_t B, int32_t H, int32_t T, int32_t c, int32_t back) {
  return (size_t)B * H * kb_cdiv_i32(T, kBK) * fused_slots(T, c, back) * kDsTileBytes;
}
// The same for a packed batch of B sequences with `total` rows in all and `max_len` rows in the longest.
size_t sa_bwd_fused_workspace_bytes_packed(int32_t B, int32_t H, int32_t total, int32_t max_len, int32_t c, int32_t back) {
  return (size_t)H * packed_tiles(total, B) * fused_slots(max_len, c, back) * kDsTileBytes;
}

int sa_bwd_fused_sm100(const kb_sa_bwd_params& p, int32_t c, int32_t back, cudaStream_t s) {
  for (void* out : {p.dq, p.dk, p.dv, p.ds_ws})
    if (reinterpret_cast<uintptr_t>(out) % 16) return KB_ERR_UNSUPPORTED;
  const size_t need = p.cu_seqlens ? sa_bwd_fused_workspace_bytes_packed(p.B, p.H, p.total_rows, p.T, c, back)
                                   : sa_bwd_fused_workspace_bytes(p.B, p.H, p.T, c, back);
  if (!p.ds_ws || p.ds_ws_bytes < need) return KB_ERR_UNSUPPORTED;
  // the delta kernel reads o and d_o rows with 16-byte loads
  for (const kb_tensor4* t : {&p.o, &p.d_o})
    if (t->stride[3] != 1 || reinterpret_cast<uintptr_t>(t->data) % 16 || t->stride[0] % 8 || t->stride[1] % 8 || t->stride[2] % 8)
      return KB_ERR_UNSUPPORTED;
  const bool bf16 = p.dtype == KB_BF16;
  if (p.cu_seqlens) {
    if (p.D == 64) return bf16 ? launch_fused<64, true, true>(p, c, back, s) : launch_fused<64, false, true>(p, c, back, s);
    if (p.D == 128) return bf16 ? launch_fused<128, true, true>(p, c, back, s) : launch_fused<128, false, true>(p, c, back, s);
    return KB_ERR_UNSUPPORTED;
  }
  if (p.D == 64) return bf16 ? launch_fused<64, true, false>(p, c, back, s) : launch_fused<64, false, false>(p, c, back, s);
  if (p.D == 128) return bf16 ? launch_fused<128, true, false>(p, c, back, s) : launch_fused<128, false, false>(p, c, back, s);
  return KB_ERR_UNSUPPORTED;
}

}  // namespace kb
