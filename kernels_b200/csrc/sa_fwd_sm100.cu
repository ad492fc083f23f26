// Streaming-attention forward for sm_100a: TMA -> shared memory -> tcgen05.mma -> TMEM.
//
// One CTA owns TWO tiles of 128 query rows (A and B, 256 consecutive rows) of one (batch, head)
// and walks the live KV tiles (128 keys each) of the streaming schedule (schedule.h); both
// q tiles use every K/V tile that is brought into shared memory, which halves the L2 traffic
// per FLOP against one q tile per CTA.  Ten warps, three roles (K and V rings two deep; output rows leave through shared memory and TMA stores):
//   warps 0-3 / 4-7  softmax of q tile A / B: thread r owns query row r of its tile (= TMEM lane
//              r).  Walks its row of a 128 x 128 block of S in TMEM twice, 64 columns at a time (row
//              maximum, then exponentials in packed fp32 arithmetic), keeps the running max / sum,
//              writes P (16-bit) back over S, rescales O when the max moved by more than 2^8,
//              writes O / LSE at the end;
//   warp 8     TMA producer (one lane): Q once, then a ring of K tiles and a ring of V tiles;
//   warp 9     MMA issuer (one lane): S = Q K^T (A, B from shared memory), O += P V
//              (A = P from TMEM, B = V from shared memory, MN-major); owns the TMEM allocation.
// MMA issue order per KV tile t:  PV_A(t-1)  S_A(t)  PV_B(t-1)  S_B(t).  While the softmax warps
// of one q tile work on their S block the tensor pipe runs the other q tile's MMAs.  MMAs
// execute in issue order, so S_A(t) may overwrite the P_A(t-1) that PV_A(t-1) reads without a
// wait, and when S_A(t) is complete so is PV_A(t-1): the softmax warps may rescale O freely.
// TMEM columns: S_A at 0, S_B at 128 (fp32; P overlays the first 64 columns of each),
// O_A at 256, O_B at 384.  One CTA per SM.
//
// The kernel is persistent: the grid is one CTA per SM and every CTA walks the work items
// (batch, head, 256-row q block) item = blockIdx.x, blockIdx.x + gridDim.x, ...  Barriers and
// TMEM are set up once; the producer runs ahead into the next item (its Q is loaded as soon as
// the last S of the current item has been issued) and the softmax warps write the current
// item's O while the MMAs of the next one already run, so the pipeline is not drained and
// refilled per item.  Consecutive items are consecutive q blocks of one (batch, head): the CTAs
// that run at the same time read neighbouring K/V rows, which keeps them in L2.
//
// Masking uses the fact that the live keys of a query row form one interval
// [max(0, i/c - back) * c, min((i/c + 1) * c, len)), which is the element form of the mask
// (i < len, j < len, 0 <= i/c - j/c <= back).  KV tiles that are live for only one of the two
// q tiles are skipped for the other.
//
// Reference semantics: src/streaming_attention/kernel.py:205-430 (online softmax in base 2,
// P cast to the input type before P V, LSE = m + log2(l)).
#include <math.h>

#include "common.cuh"
#include <type_traits>

#include "sm100_ptx.cuh"
#include "sm100_host.h"
#include "tiles.h"

namespace kb {
#ifdef KB_TRACE_FWD
// Debug build only: where the MMA thread and one softmax thread of CTA 60 spend their clocks; read back by
// kb_debug_trace_fwd().  [0..15] MMA thread, [16..31] softmax thread (q tile A, row 0).
__device__ long long g_fwtrace[32];
#define KB_FACC(i) do { const long long tn_ = clock64(); acc_t[i] += tn_ - tl; tl = tn_; } while (0)
#else
#define KB_FACC(i) do { } while (0)
#endif
namespace {

using namespace sm100;

constexpr int kBM = tiles::kFwdQRows;  // rows of one q tile
constexpr int kQTiles = tiles::kFwdQTiles;
constexpr int kBN = tiles::kFwdKeys;
constexpr int kStagesK = tiles::kFwdStagesK, kStagesV = tiles::kFwdStagesV;
static_assert(kBM == 128 && kBN == 128 && kQTiles == 2, "the TMEM column map and the warp roles assume two 128 x 128 score blocks");
constexpr int kThreads = (kQTiles * 4 + 2) * 32;
constexpr int kProducerWarp = kQTiles * 4, kMmaWarp = kQTiles * 4 + 1;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256;  // + 128 * q tile
// Lazy rescale: the reference maximum of a row is only moved when the new maximum exceeds it by this many
// log2 units, so P can reach 2^threshold.  16-bit P has the range for 2^8; e4m3 P (largest value 448) is formed
// as p * 2^kFp8POffset * (v scale / largest v scale) with threshold + offset = 8, i.e. at most 256.
constexpr float kRescaleThreshold = 8.f, kRescaleThresholdFp8 = 3.f, kFp8POffset = 5.f;

struct FwdArgs {
  void* o;
  float* lse;
  const int32_t* lens;
  int64_t lens_stride;
  int64_t o_sb, o_sh, o_st, lse_sb, lse_sh;  // element strides of o (b, h, t) and of lse (b, h)
  int32_t B, H, T, c, back;
  int32_t q_start;  // the query rows are the positions [q_start, T): row r of q / o / lse is position q_start + r
  // Packed batch: sequence b owns the rows [cu[b], cu[b + 1]) of tensors with ONE batch entry (the maps' batch
  // extent is 1, o_sb = lse_sb = 0) and T is the longest sequence.  NULL: the padded layout.
  const int32_t* cu;
  KbFastDiv fd_qblocks, fd_H, fd_c, fd_group;  // division by ceil(T / 256), H, c and H / H_kv (query heads per K/V head)
  float scale_log2;
  int32_t* status;
  // 8-bit (e4m3) inputs only: one dequantisation scale per tile of 128 rows of q [B, H, n128], k and v
  // [B, H_kv, n128], and the largest v scale of every key/value head [B, H_kv]
  const float* q_scale;
  const float* k_scale;
  const float* v_scale;
  const float* v_scale_max;
  int32_t n128, Hk;
};

template <int D>
struct alignas(1024) FwdSmem {
  uint8_t q[kQTiles][kBM * D * 2];
  uint8_t k[kStagesK][kBN * D * 2];
  uint8_t v[kStagesV][kBN * D * 2];
  uint8_t o_stage[kQTiles][kBM * 128];  // one 64-column panel of a q tile's output on its way to a TMA store
  uint64_t q_full, k_full[kStagesK], k_empty[kStagesK], v_full[kStagesV], v_empty[kStagesV];
  uint64_t q_empty, s_ready[kQTiles], p_ready[kQTiles], o_done[kQTiles], o_free[kQTiles];
  uint32_t tmem_base;
  int abort_flag;
};

enum WaitSite { kWaitQ = 1, kWaitQEmpty, kWaitOFree, kWaitKEmpty, kWaitVEmpty, kWaitKFull, kWaitVFull, kWaitSReady, kWaitPReady, kWaitEpilogue };
constexpr int kErrSmemAlign = 11;

// One 128 x 128 block of scores for the thread's row, in two passes over the row in TMEM, 64 columns at a
// time, so that at most 64 scores are live in registers (holding all 128 leaves the softmax warps no register to
// spare at the 168 the launch gives them, and every spill sits on the kernel's critical chain).
// Pass 1 (softmax_row_max): the row maximum of the masked scores.  kMasked = false is the fast path for blocks
// in which every element of the warp's rows is live.
template <bool kMasked>
__device__ __forceinline__ float softmax_row_max(uint32_t t_s, int k0, int lo, int hi) {
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    uint32_t s[64];
    tmem_ld32(t_s + half * 64, reinterpret_cast<uint32_t(&)[32]>(s[0]));
    tmem_ld32(t_s + half * 64 + 32, reinterpret_cast<uint32_t(&)[32]>(s[32]));
    tmem_wait_ld();
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const int c0 = k0 + half * 64 + cc * 32;
      // a 32-column group that is live for every row of the warp needs no select, one that is masked for every
      // row contributes nothing (chunk boundaries that are multiples of 32 never leave a mixed group)
      const bool all_live = !kMasked || __all_sync(0xffffffffu, lo <= c0 && c0 + 32 <= hi);
      const bool all_dead = kMasked && __all_sync(0xffffffffu, c0 + 32 <= lo || c0 >= hi);
      if (all_dead) continue;
      // 3-input max: two scores per instruction
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = cc * 32 + i + 2 * e;
          float a = __uint_as_float(s[j]), b = __uint_as_float(s[j + 1]);
          if (!all_live) {
            a = (c0 + i + 2 * e >= lo && c0 + i + 2 * e < hi) ? a : -INFINITY;
            b = (c0 + i + 2 * e + 1 >= lo && c0 + i + 2 * e + 1 < hi) ? b : -INFINITY;
          }
          mx[e] = fmax3(mx[e], a, b);
        }
      }
    }
  }
  return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}

// Pass 2 (softmax_exp_half): P = 2^(S scale - m) for the 64 columns [64 half, 64 half + 64) of the row, 16-bit,
// into TMEM over S (P of columns 32 j .. 32 j + 31 lands on columns 16 j .. 16 j + 15: the second half of P
// overwrites only scores of the first half, which are in registers by then); the row sum goes into `sum`.
// FP8: P is written as e4m3, four values per TMEM column (64 keys = 16 columns at 16 half), for the 8-bit P V.
template <bool BF16, bool kMasked, bool FP8>
__device__ __forceinline__ void softmax_exp_half(uint32_t t_s, int half, float scale, float m_used, int k0, int lo, int hi,
                                                 float (&sum)[4]) {
  const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
  // packed fp32 arithmetic: one FMA and one add per PAIR of scores
  const uint64_t scale2 = f2_pack(scale, scale), negm2 = f2_pack(-m_safe, -m_safe);
  uint64_t sum01 = f2_pack(sum[0], sum[1]), sum23 = f2_pack(sum[2], sum[3]);
  uint32_t s[64];
  tmem_ld32(t_s + half * 64, reinterpret_cast<uint32_t(&)[32]>(s[0]));
  tmem_ld32(t_s + half * 64 + 32, reinterpret_cast<uint32_t(&)[32]>(s[32]));
  tmem_wait_ld();
#pragma unroll
  for (int cc = 0; cc < 2; ++cc) {
    const int c0 = k0 + half * 64 + cc * 32;
    const bool all_live = !kMasked || __all_sync(0xffffffffu, lo <= c0 && c0 + 32 <= hi);
    const bool all_dead = kMasked && __all_sync(0xffffffffu, c0 + 32 <= lo || c0 >= hi);
    uint32_t pk[16];
    if (all_dead) {
#pragma unroll
      for (int i = 0; i < 16; ++i) pk[i] = 0u;
      if (FP8) tmem_st8(t_s + (half * 2 + cc) * 8, reinterpret_cast<const uint32_t(&)[8]>(pk[0]));
      else tmem_st16(t_s + (half * 2 + cc) * 16, pk);
      continue;
    }
    float pf[FP8 ? 32 : 1];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float s0 = __uint_as_float(s[cc * 32 + 2 * i]), s1 = __uint_as_float(s[cc * 32 + 2 * i + 1]);
      if (!all_live) {
        s0 = (c0 + 2 * i >= lo && c0 + 2 * i < hi) ? s0 : -INFINITY;
        s1 = (c0 + 2 * i + 1 >= lo && c0 + 2 * i + 1 < hi) ? s1 : -INFINITY;
      }
      const uint64_t x = f2_fma(f2_pack(s0, s1), scale2, negm2);
      float x0, x1;
      f2_unpack(x, x0, x1);
      const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
      if (i & 1) sum23 = f2_add(sum23, f2_pack(p0, p1)); else sum01 = f2_add(sum01, f2_pack(p0, p1));
      if (FP8) {
        pf[2 * i] = p0;
        pf[2 * i + 1] = p1;
      } else {
        pk[i] = pack16x2<BF16>(p0, p1);
      }
    }
    if (FP8) {
#pragma unroll
      for (int i = 0; i < 8; ++i) pk[i] = pack_e4m3x4(pf[4 * i], pf[4 * i + 1], pf[4 * i + 2], pf[4 * i + 3]);
      tmem_st8(t_s + (half * 2 + cc) * 8, reinterpret_cast<const uint32_t(&)[8]>(pk[0]));
    } else {
      tmem_st16(t_s + (half * 2 + cc) * 16, pk);
    }
  }
  f2_unpack(sum01, sum[0], sum[1]);
  f2_unpack(sum23, sum[2], sum[3]);
}

// PACKED: one launch over a packed batch (FwdArgs::cu).  FP8: q, k, v are e4m3 with per-tile scales, both matmuls
// run as kind::f8f6f4 (half the instructions), the output is 16-bit (BF16 selects which).
// The same block in ONE pass for head dim 64, where the registers allow it (the epilogue holds 64 output columns,
// not 128) and where it matters: with half the matmul work per block the softmax warps set the pace, and the
// second walk over TMEM is time on their chain.  Loads the row's 128 scores once; returns the row maximum.
template <bool kMasked>
__device__ __forceinline__ float softmax_load_row_max(uint32_t t_s, uint32_t (&s)[kBN], bool (&dead)[kBN / 32], int k0, int lo, int hi) {
#pragma unroll
  for (int cc = 0; cc < kBN / 32; ++cc) tmem_ld32(t_s + cc * 32, reinterpret_cast<uint32_t(&)[32]>(s[cc * 32]));
  tmem_wait_ld();
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int cc = 0; cc < kBN / 32; ++cc) {
    const int c0 = k0 + cc * 32;
    const bool all_live = !kMasked || __all_sync(0xffffffffu, lo <= c0 && c0 + 32 <= hi);
    dead[cc] = kMasked && __all_sync(0xffffffffu, c0 + 32 <= lo || c0 >= hi);
    if (dead[cc]) continue;
    if (!all_live) {
#pragma unroll
      for (int i = 0; i < 32; ++i) s[cc * 32 + i] = (c0 + i >= lo && c0 + i < hi) ? s[cc * 32 + i] : 0xff800000u;  // -inf
    }
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        mx[e] = fmax3(mx[e], __uint_as_float(s[cc * 32 + i + 2 * e]), __uint_as_float(s[cc * 32 + i + 2 * e + 1]));
    }
  }
  return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}
// ... and P = 2^(S scale - m) from the registers, 16-bit, into TMEM over S; the row sum goes into `sum`.
template <bool BF16, bool kMasked>
__device__ __forceinline__ void softmax_exp_held(uint32_t t_s, const uint32_t (&s)[kBN], const bool (&dead)[kBN / 32], float scale,
                                                 float m_used, float (&sum)[4]) {
  const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
#pragma unroll
  for (int cc = 0; cc < kBN / 32; ++cc) {
    uint32_t pk[16];
    if (kMasked && dead[cc]) {
#pragma unroll
      for (int i = 0; i < 16; ++i) pk[i] = 0u;
      tmem_st16(t_s + cc * 16, pk);
      continue;
    }
    // scalar arithmetic here: with 128 scores held, the register pairs of the packed form do not fit
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
}

// FAST: the instance for chunk lengths that are multiples of the work item's 256 rows, where the two q tiles of
// every item lie in one chunk and walk the same key tiles: the MMA thread then runs such items through a
// straight-line schedule (first / inner / last step written out, nothing worked out per step).  Other chunk
// lengths are built without it (the extra code measured 1.5 % slower there).
template <int D, bool BF16, bool PACKED, bool FP8, bool FAST>
__global__ void __launch_bounds__(kThreads, 1)
sa_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, const FwdArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  FwdSmem<D>& sm = *reinterpret_cast<FwdSmem<D>*>(smem_raw);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T = a.T;
  const int n_qblocks = kb_cdiv_i32(T - a.q_start, kBM * kQTiles);
  const int n_items = a.B * a.H * n_qblocks;

  if (smem_u32(smem_raw) & 1023u) {
    // swizzled operand tiles need a 1024-byte aligned base: report instead of computing garbage
    if (threadIdx.x == 0 && a.status) {
      atomicExch(a.status, KB_ERR_DEVICE_TIMEOUT);
      atomicExch(a.status + 1, kErrSmemAlign);
    }
    return;
  }

  // One work item: a 256-row q block of one (batch, head) with the live KV tiles of its two
  // q tiles and of the block (their union: both ranges are contiguous, B's starts and ends no
  // earlier than A's, and they touch or overlap).  Every role decodes items the same way.
  struct Item {
    int b, h, q0, len;
    int row0;  // first row of the sequence in the tensor maps (packed batch: cu[b], batch coordinate 0)
    KbTileRange kr[kQTiles];
    bool act[kQTiles];
    int u_begin, u_end;
  };
  auto decode = [&](int item) {
    Item it;
    const int bh = kb_fastdiv(item, a.fd_qblocks), qb = item - bh * n_qblocks;
    it.b = kb_fastdiv(bh, a.fd_H);
    it.h = bh - it.b * a.H;
    it.q0 = a.q_start + qb * (kBM * kQTiles);
    it.len = a.lens ? kb_clamp_len(a.lens[(int64_t)it.b * a.lens_stride], T) : T;
    it.row0 = 0;
    if (PACKED) {
      it.row0 = a.cu[it.b];
      it.len = kb_min_i32(a.cu[it.b + 1] - it.row0, T);
    }
#pragma unroll
    for (int x = 0; x < kQTiles; ++x) {
      it.kr[x] = kb_fwd_kv_range_fd(it.q0 + x * kBM, kBM, kBN, it.len, a.c, a.back, a.fd_c);
      it.act[x] = it.kr[x].begin < it.kr[x].end;
    }
    it.u_begin = it.act[0] ? it.kr[0].begin : it.kr[1].begin;
    it.u_end = it.act[1] ? it.kr[1].end : it.kr[0].end;
    return it;
  };

  if (threadIdx.x == 0) {
    mbar_init(&sm.q_full, 1);
    mbar_init(&sm.q_empty, 1);
    for (int s = 0; s < kStagesK; ++s) {
      mbar_init(&sm.k_full[s], 1);
      mbar_init(&sm.k_empty[s], 1);
    }
    for (int s = 0; s < kStagesV; ++s) {
      mbar_init(&sm.v_full[s], 1);
      mbar_init(&sm.v_empty[s], 1);
    }
    for (int x = 0; x < kQTiles; ++x) {
      mbar_init(&sm.s_ready[x], 1);
      mbar_init(&sm.p_ready[x], kBM);
      mbar_init(&sm.o_done[x], 1);
      mbar_init(&sm.o_free[x], kBM);
    }
    sm.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kMmaWarp) tmem_alloc(&sm.tmem_base, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const WaitCtx ctx{&sm.abort_flag, a.status};
  constexpr uint32_t kPanelBytes = 128 * 128;  // 128 rows x 128 bytes
  constexpr uint32_t kTileBytes = 128 * D * (FP8 ? 1 : 2);
  constexpr int kPanels = FP8 ? D / 128 : D / 64;  // 128-byte panels of an input row
  constexpr int kPanelElems = FP8 ? 128 : 64;
  constexpr int kOutPanels = D / 64;               // of a 16-bit output row

  // Barrier phases are counted over the whole life of the CTA: kc / vc = K / V tiles so far,
  // na = items with at least one live q tile so far, per q tile: tiles and items so far.
  if (warp == kProducerWarp) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      int kc = 0, vc = 0, na = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
        const Item it = decode(item);
        if (!it.act[0] && !it.act[1]) continue;
        // the Q buffers are free once every S of the previous item has been issued and has run
        if (na > 0 && !mbar_wait(&sm.q_empty, (na - 1) & 1, ctx, kWaitQEmpty)) break;
        mbar_expect_tx(&sm.q_full, (it.act[0] ? kTileBytes : 0) + (it.act[1] ? kTileBytes : 0));
#pragma unroll
        for (int x = 0; x < kQTiles; ++x) {
          if (!it.act[x]) continue;
#pragma unroll
          for (int p = 0; p < kPanels; ++p)
            tma_load_4d(sm.q[x] + p * kPanelBytes, &tm_q, &sm.q_full, p * kPanelElems, it.row0 + it.q0 - a.q_start + x * kBM, it.h, PACKED ? 0 : it.b);
        }
        const int h_kv = kb_fastdiv(it.h, a.fd_group);  // the K/V head this query head reads
        for (int t = it.u_begin; t < it.u_end; ++t, ++kc, ++vc) {
          const int sk = kc % kStagesK, sv = vc % kStagesV;
          const int k0 = t * kBN;
          if (kc >= kStagesK && !mbar_wait(&sm.k_empty[sk], ((kc / kStagesK) - 1) & 1, ctx, kWaitKEmpty)) { ok = false; break; }
          mbar_expect_tx(&sm.k_full[sk], kTileBytes);
#pragma unroll
          for (int p = 0; p < kPanels; ++p) tma_load_4d(sm.k[sk] + p * kPanelBytes, &tm_k, &sm.k_full[sk], p * kPanelElems, it.row0 + k0, h_kv, PACKED ? 0 : it.b);
          if (vc >= kStagesV && !mbar_wait(&sm.v_empty[sv], ((vc / kStagesV) - 1) & 1, ctx, kWaitVEmpty)) { ok = false; break; }
          mbar_expect_tx(&sm.v_full[sv], kTileBytes);
#pragma unroll
          for (int p = 0; p < kPanels; ++p) tma_load_4d(sm.v[sv] + p * kPanelBytes, &tm_v, &sm.v_full[sv], p * kPanelElems, it.row0 + k0, h_kv, PACKED ? 0 : it.b);
        }
        ++na;
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = FP8 ? make_idesc_e4m3(kBM, kBN, false, false) : make_idesc(BF16, kBM, kBN, false, false);
      constexpr uint32_t idesc_pv = FP8 ? make_idesc_e4m3(kBM, D, false, true) : make_idesc(BF16, kBM, D, false, true);
      int kbase = 0, na = 0;            // K (= V) tiles of earlier items, live items so far
      int tiles_x[kQTiles] = {0, 0};    // S / P blocks of q tile x so far
      int items_x[kQTiles] = {0, 0};    // items in which q tile x was live so far
      bool ok = true;
#ifdef KB_TRACE_FWD
      long long acc_t[10] = {0};
      long long tl = clock64();
#endif
      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
        const Item it = decode(item);
        if (!it.act[0] && !it.act[1]) continue;
        KB_FACC(0);
        if (!mbar_wait(&sm.q_full, na & 1, ctx, kWaitQ)) break;
        KB_FACC(1);
        // Step s issues, per q tile x:  PV_x(s - 1) then S_x(s), each q tile walking its own key tiles in order.
        // When tile B's range starts d key tiles after tile A's (chunks shorter than the 256-row item: the two q
        // tiles then see different windows) and the K / V rings can hold d + 1 tiles, both q tiles start at step
        // 0 on their own first tile ("skewed": B works d key tiles ahead of A), so that every step carries both
        // q tiles and each one's softmax overlaps the other's MMAs; otherwise B starts at step d on the tile A is
        // on.  Either way a q tile sees its key tiles in the same order, so the results are the same bits.
        const int n_x[kQTiles] = {it.act[0] ? it.kr[0].end - it.kr[0].begin : 0, it.act[1] ? it.kr[1].end - it.kr[1].begin : 0};
        const int d = (it.act[0] && it.act[1]) ? it.kr[1].begin - it.kr[0].begin : 0;
        const int first_x[kQTiles] = {0, d < kStagesK && d < kStagesV ? 0 : d};
        const int n_steps = kb_max_i32(first_x[0] + n_x[0], first_x[1] + n_x[1]);
        // the step at which q tile x visits key tile t (only meaningful for t inside its range)
        auto step_of = [&](int x, int t) { return first_x[x] + t - it.kr[x].begin; };
        // q tile x is the last of the item to use key tile t (in a matmul of the kind issued at its step)
        auto last_user = [&](int x, int t) {
          const int y = 1 - x;
          if (!(it.act[y] && t >= it.kr[y].begin && t < it.kr[y].end)) return true;
          const int sx = step_of(x, t), sy = step_of(y, t);
          return sx > sy || (sx == sy && x > y);
        };
        // O_x (+)= P_x V of the q tile's lx-th key tile, V being ring tile vi (counted over the CTA's life)
        auto issue_pv = [&](auto first_c, auto last_c, int x, int vi, bool release_v) -> bool {
          constexpr bool kFirst = decltype(first_c)::value, kLast = decltype(last_c)::value;  // of the q tile's key tiles
          const int sv = vi % kStagesV;
          const int px = tiles_x[x] - 1;  // P block consumed now = last S block issued for x
          KB_FACC(2);
          if (!mbar_wait(&sm.p_ready[x], px & 1, ctx, kWaitPReady)) return false;
          KB_FACC(3 + x);
          if (!mbar_wait(&sm.v_full[sv], (vi / kStagesV) & 1, ctx, kWaitVFull)) return false;
          KB_FACC(5);
          // the first P V of an item overwrites O: the softmax warps must have read the old one
          if (kFirst && items_x[x] > 0 && !mbar_wait(&sm.o_free[x], (items_x[x] - 1) & 1, ctx, kWaitOFree)) return false;
          tc_fence_after();
          // short issue loops (four instructions per trip, descriptor low words stepped by adds): the
          // scalar work between two MMAs is what the tensor pipe waits for
          uint32_t p_col = tmem + kColS + x * 128, v_lo = desc_lo_mnmajor(smem_u32(sm.v[sv]), kPanelBytes);
          if (FP8) {
            // 128 keys = four instructions of 32 keys: 8 packed columns of P, 32 rows (4096 bytes) of V each
#pragma unroll
            for (int i = 0; i < 4; ++i)
              mma_ts_lo_f8(tmem + kColO + x * 128, p_col + 8 * i, v_lo + i * (4096 >> 4), idesc_pv, !kFirst || i > 0);
          } else {
#pragma unroll 1
            for (int h = 0; h < kBN / 64; ++h, p_col += 32, v_lo += 4 * (2048 >> 4)) {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                mma_ts_lo(tmem + kColO + x * 128, p_col + 8 * i, v_lo + i * (2048 >> 4), idesc_pv, !kFirst || h > 0 || i > 0);
            }
          }
          if (release_v) mma_commit(&sm.v_empty[sv]);  // V is free once the last q tile that uses it has consumed it
          if (kLast) mma_commit(&sm.o_done[x]);
          KB_FACC(6);
          return true;
        };
        // S_x = Q_x K^T, K being ring tile ki
        auto issue_s = [&](int x, int ki, bool release_k) -> bool {
          const int sk = ki % kStagesK;
          KB_FACC(2);
          if (!mbar_wait(&sm.k_full[sk], (ki / kStagesK) & 1, ctx, kWaitKFull)) return false;
          KB_FACC(7);
          tc_fence_after();
          uint32_t q_lo = desc_lo_kmajor(smem_u32(sm.q[x])), k_lo = desc_lo_kmajor(smem_u32(sm.k[sk]));
#pragma unroll 1
          for (int h = 0; h < kPanels; ++h, q_lo += kPanelBytes >> 4, k_lo += kPanelBytes >> 4) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {  // 32 bytes of every row per instruction: 16 16-bit or 32 8-bit elements
              if (FP8) mma_ss_lo_f8(tmem + kColS + x * 128, q_lo + 2 * i, k_lo + 2 * i, idesc_qk, h > 0 || i > 0);
              else mma_ss_lo(tmem + kColS + x * 128, q_lo + 2 * i, k_lo + 2 * i, idesc_qk, h > 0 || i > 0);
            }
          }
          if (release_k) mma_commit(&sm.k_empty[sk]);
          mma_commit(&sm.s_ready[x]);
          ++tiles_x[x];
          KB_FACC(8);
          return true;
        };
        if (FAST && it.act[0] && it.act[1] && d == 0 && n_x[0] == n_x[1]) {
          // Both q tiles on the same key tiles at the same steps: ring tile kbase + i is the i-th key tile of both,
          // tile B its last user.  First, inner and last step are written out.
          using Yes = std::true_type;
          using No = std::false_type;
          const int n = n_x[0];
          ok = issue_s(0, kbase, false) && issue_s(1, kbase, true);
          if (n == 1) {
            mma_commit(&sm.q_empty);  // every S of this item has been issued
            ok = ok && issue_pv(Yes{}, Yes{}, 0, kbase, false) && issue_pv(Yes{}, Yes{}, 1, kbase, true);
          } else {
            ok = ok && issue_pv(Yes{}, No{}, 0, kbase, false) && issue_s(0, kbase + 1, false) &&
                 issue_pv(Yes{}, No{}, 1, kbase, true) && issue_s(1, kbase + 1, true);
            if (n == 2) mma_commit(&sm.q_empty);
            for (int step = 2; ok && step < n; ++step) {
              ok = issue_pv(No{}, No{}, 0, kbase + step - 1, false) && issue_s(0, kbase + step, false) &&
                   issue_pv(No{}, No{}, 1, kbase + step - 1, true) && issue_s(1, kbase + step, true);
              if (step == n - 1) mma_commit(&sm.q_empty);
            }
            ok = ok && issue_pv(No{}, Yes{}, 0, kbase + n - 1, false) && issue_pv(No{}, Yes{}, 1, kbase + n - 1, true);
          }
        } else {
          // (the same two issue sequences, written out: through the lambdas this path measured 3-4 % slower)
          for (int step = 0; ok && step <= n_steps; ++step) {
  #pragma unroll
            for (int x = 0; x < kQTiles; ++x) {
              const bool pv_live = it.act[x] && step - 1 >= first_x[x] && step - 1 < first_x[x] + n_x[x];
              const bool s_live = it.act[x] && step >= first_x[x] && step < first_x[x] + n_x[x];
              if (pv_live) {
                const int lx = step - 1 - first_x[x];  // index within this q tile's range
                const int u = it.kr[x].begin + lx, vi = kbase + (u - it.u_begin), sv = vi % kStagesV;
                const int px = tiles_x[x] - 1;  // P block consumed now = last S block issued for x
                KB_FACC(2);
                if (!mbar_wait(&sm.p_ready[x], px & 1, ctx, kWaitPReady)) { ok = false; break; }
                KB_FACC(3 + x);
                if (!mbar_wait(&sm.v_full[sv], (vi / kStagesV) & 1, ctx, kWaitVFull)) { ok = false; break; }
                KB_FACC(5);
                // the first P V of an item overwrites O: the softmax warps must have read the old one
                if (lx == 0 && items_x[x] > 0 && !mbar_wait(&sm.o_free[x], (items_x[x] - 1) & 1, ctx, kWaitOFree)) { ok = false; break; }
                tc_fence_after();
                // short issue loops (four instructions per trip, descriptor low words stepped by adds): the
                // scalar work between two MMAs is what the tensor pipe waits for
                uint32_t p_col = tmem + kColS + x * 128, v_lo = desc_lo_mnmajor(smem_u32(sm.v[sv]), kPanelBytes);
                if (FP8) {
                  // 128 keys = four instructions of 32 keys: 8 packed columns of P, 32 rows (4096 bytes) of V each
  #pragma unroll
                  for (int i = 0; i < 4; ++i)
                    mma_ts_lo_f8(tmem + kColO + x * 128, p_col + 8 * i, v_lo + i * (4096 >> 4), idesc_pv, lx > 0 || i > 0);
                } else {
  #pragma unroll 1
                  for (int h = 0; h < kBN / 64; ++h, p_col += 32, v_lo += 4 * (2048 >> 4)) {
  #pragma unroll
                    for (int i = 0; i < 4; ++i)
                      mma_ts_lo(tmem + kColO + x * 128, p_col + 8 * i, v_lo + i * (2048 >> 4), idesc_pv, lx > 0 || h > 0 || i > 0);
                  }
                }
                // V_u is free once the last q tile that uses it has consumed it
                if (last_user(x, u)) mma_commit(&sm.v_empty[sv]);
                if (u == it.kr[x].end - 1) mma_commit(&sm.o_done[x]);
                KB_FACC(6);
              }
              if (s_live) {
                const int t = it.kr[x].begin + (step - first_x[x]);
                const int ki = kbase + (t - it.u_begin), sk = ki % kStagesK;
                KB_FACC(2);
                if (!mbar_wait(&sm.k_full[sk], (ki / kStagesK) & 1, ctx, kWaitKFull)) { ok = false; break; }
                KB_FACC(7);
                tc_fence_after();
                uint32_t q_lo = desc_lo_kmajor(smem_u32(sm.q[x])), k_lo = desc_lo_kmajor(smem_u32(sm.k[sk]));
  #pragma unroll 1
                for (int h = 0; h < kPanels; ++h, q_lo += kPanelBytes >> 4, k_lo += kPanelBytes >> 4) {
  #pragma unroll
                  for (int i = 0; i < 4; ++i) {  // 32 bytes of every row per instruction: 16 16-bit or 32 8-bit elements
                    if (FP8) mma_ss_lo_f8(tmem + kColS + x * 128, q_lo + 2 * i, k_lo + 2 * i, idesc_qk, h > 0 || i > 0);
                    else mma_ss_lo(tmem + kColS + x * 128, q_lo + 2 * i, k_lo + 2 * i, idesc_qk, h > 0 || i > 0);
                  }
                }
                if (last_user(x, t)) mma_commit(&sm.k_empty[sk]);
                mma_commit(&sm.s_ready[x]);
                ++tiles_x[x];
                KB_FACC(8);
              }
            }
            if (step == n_steps - 1) mma_commit(&sm.q_empty);  // every S of this item has been issued
          }
        }
        kbase += it.u_end - it.u_begin;
        ++na;
#pragma unroll
        for (int x = 0; x < kQTiles; ++x) items_x[x] += it.act[x] ? 1 : 0;
      }
#ifdef KB_TRACE_FWD
      if (blockIdx.x == 60)
        for (int i = 0; i < 10; ++i) g_fwtrace[i] = acc_t[i];
#endif
    }
  } else {
    // ------------------------------ softmax + epilogue ------------------------------
    const int x = warp >> 2;  // q tile of this warpgroup
    const int row = (warp & 3) * 32 + lane;
    const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t t_s = t_lane + kColS + x * 128, t_o = t_lane + kColO + x * 128;
    const float scale_base = a.scale_log2;
    int tiles = 0, items = 0;  // S blocks / live items of this q tile so far
    bool ok = true;
#ifdef KB_TRACE_FWD
    long long acc_t[8] = {0};
    long long tl = clock64();
#endif
    for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
      const Item it = decode(item);
      const int qi = it.q0 + x * kBM + row;
      const int orow = it.row0 + qi - a.q_start;  // this thread's row of o and lse
      uint16_t* o_row = static_cast<uint16_t*>(a.o) + it.b * a.o_sb + it.h * a.o_sh + orow * a.o_st;
      float* lse_row = a.lse ? a.lse + it.b * a.lse_sb + it.h * a.lse_sh + orow : nullptr;
      if (!it.act[x]) {
        // this q tile lies wholly in the padding: its rows are zeros
        if (qi < (PACKED ? it.len : T)) {  // a packed batch has no padding rows
          uint4* dst = reinterpret_cast<uint4*>(o_row);
#pragma unroll
          for (int i = 0; i < D * 2 / 16; ++i) dst[i] = make_uint4(0, 0, 0, 0);
          if (lse_row) *lse_row = 0.f;
        }
        continue;
      }
      const int n_tiles = it.kr[x].end - it.kr[x].begin;
      int lo = 0, hi = 0;
      if (qi < it.len) {
        const int qc = kb_fastdiv(qi, a.fd_c);
        lo = kb_max_i32(0, qc - a.back) * a.c;
        const int64_t h64 = (int64_t)(qc + 1) * a.c;
        hi = h64 < it.len ? (int)h64 : it.len;
      }
      float m_used = -INFINITY, l = 0.f;
      // 8-bit inputs: the scores of a tile carry the scales of its q and k tiles (folded into the softmax scale);
      // P of a tile is formed as p * 2^kFp8POffset * (v scale of the tile) / (largest v scale of the head), which
      // uses e4m3's range and lets one accumulator add tiles with different v scales: the factor enters the
      // exponent (p_off) and is taken out of the tile's row sum again; O is divided by it at the end.
      float q_sc = 1.f, v_inv_max = 1.f, v_max = 1.f;
      const float* k_sc_row = nullptr;
      const float* v_sc_row = nullptr;
      if (FP8) {
        const int h_kv = kb_fastdiv(it.h, a.fd_group);
        q_sc = a.q_scale[((int64_t)it.b * a.H + it.h) * a.n128 + ((it.q0 + x * kBM) >> 7)];
        k_sc_row = a.k_scale + ((int64_t)it.b * a.Hk + h_kv) * a.n128;
        v_sc_row = a.v_scale + ((int64_t)it.b * a.Hk + h_kv) * a.n128;
        v_max = a.v_scale_max[(int64_t)it.b * a.Hk + h_kv];
        v_inv_max = 1.f / v_max;
      }

      for (int lx = 0; lx < n_tiles; ++lx, ++tiles) {
        const int k0 = (it.kr[x].begin + lx) * kBN;
        float scale = scale_base, p_off = 0.f;
        if (FP8) {
          scale = scale_base * q_sc * k_sc_row[k0 >> 7];
          p_off = kFp8POffset + log2f(fmaxf(v_sc_row[k0 >> 7] * v_inv_max, 9.5367431640625e-7f));
        }
        KB_FACC(0);
        ok = __all_sync(0xffffffffu, mbar_wait(&sm.s_ready[x], tiles & 1, ctx, kWaitSReady));
        if (!ok) break;
        tc_fence_after();
        KB_FACC(1);
        const bool warp_full = __all_sync(0xffffffffu, lo <= k0 && k0 + kBN <= hi);
        constexpr bool kHold = (D == 64) && !FP8;  // one pass with the row's scores held in registers
        uint32_t s_held[kHold ? kBN : 1];
        bool dead_held[kBN / 32];
        float row_max;
        if (kHold) {
          row_max = warp_full ? softmax_load_row_max<false>(t_s, reinterpret_cast<uint32_t(&)[kBN]>(s_held), dead_held, k0, lo, hi)
                              : softmax_load_row_max<true>(t_s, reinterpret_cast<uint32_t(&)[kBN]>(s_held), dead_held, k0, lo, hi);
        } else {
          row_max = warp_full ? softmax_row_max<false>(t_s, k0, lo, hi) : softmax_row_max<true>(t_s, k0, lo, hi);
        }
        const float m_new = fmaxf(m_used, row_max * scale);
        // lazy rescale: keep the old reference maximum unless the new one is larger by more than the threshold
        const bool need = m_new > m_used + (FP8 ? kRescaleThresholdFp8 : kRescaleThreshold);
        float alpha = 1.f;
        if (need) {
          alpha = ex2_approx(m_used - m_new);
          m_used = m_new;
          l *= alpha;
        }
        KB_FACC(2);
        KB_FACC(3);
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
        const float m_exp = m_used - p_off;  // 2^(s scale - m_exp) = p * 2^p_off
        if (kHold) {
          if (warp_full) softmax_exp_held<BF16, false>(t_s, reinterpret_cast<const uint32_t(&)[kBN]>(s_held), dead_held, scale, m_exp, sum);
          else softmax_exp_held<BF16, true>(t_s, reinterpret_cast<const uint32_t(&)[kBN]>(s_held), dead_held, scale, m_exp, sum);
        } else {
          if (warp_full) softmax_exp_half<BF16, false, FP8>(t_s, 0, scale, m_exp, k0, lo, hi, sum);
          else softmax_exp_half<BF16, true, FP8>(t_s, 0, scale, m_exp, k0, lo, hi, sum);
          if (warp_full) softmax_exp_half<BF16, false, FP8>(t_s, 1, scale, m_exp, k0, lo, hi, sum);
          else softmax_exp_half<BF16, true, FP8>(t_s, 1, scale, m_exp, k0, lo, hi, sum);
        }
        // the rescale of O comes after the exponentials: the row's scores are dead by now, which keeps the
        // registers of the two from being live together
        if (lx > 0 && __any_sync(0xffffffffu, need)) {
          // S(lx) is complete, so the P V of the previous tile (issued before it) is too: O is idle
#pragma unroll
          for (int cc = 0; cc < D / 32; ++cc) {
            uint32_t r[32];
            tmem_ld32(t_o + cc * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(t_o + cc * 32, r);
          }
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&sm.p_ready[x]);
        if (FP8) l += ((sum[0] + sum[1]) + (sum[2] + sum[3])) * ex2_approx(-p_off);
        else l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
        KB_FACC(4);
      }
      if (!ok) break;
      KB_FACC(0);

      ok = __all_sync(0xffffffffu, mbar_wait(&sm.o_done[x], items & 1, ctx, kWaitEpilogue));
      if (!ok) break;
      KB_FACC(5);
      ++items;
      tc_fence_after();
      // pull the whole O row out of TMEM, release the accumulator to the next item, then store
      uint32_t r[D];
#pragma unroll
      for (int cc = 0; cc < D / 32; ++cc) tmem_ld32(t_o + cc * 32, reinterpret_cast<uint32_t(&)[32]>(r[cc * 32]));
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&sm.o_free[x]);
      const bool valid = qi < it.len;
      const float inv = valid ? (FP8 ? v_max * exp2f(-kFp8POffset) / l : 1.f / l) : 0.f;
      // The rows leave through shared memory and a TMA store, one 64-column panel at a time (row = 128
      // bytes, 128-byte swizzle).  Plain 16-byte stores of a 256-byte row per thread touch 32 different
      // lines per instruction and held the softmax warps for several thousand clocks per item.  Rows past
      // the end of the tensor are clipped by the store; rows past `len` are zeros (inv = 0).
      uint8_t* stage = sm.o_stage[x] + row * 128;
      if (PACKED && it.q0 + x * kBM + kBM > it.len) {
        // packed batch, last tile of a sequence: the rows below belong to the next sequence, so no box store;
        // every thread writes its own row (one such tile per sequence and head)
        if (valid) {
          uint4* dst = reinterpret_cast<uint4*>(o_row);
#pragma unroll
          for (int j = 0; j < D / 8; ++j) {
            const int e = 8 * j;
            uint4 w;
            w.x = pack16x2<BF16>(__uint_as_float(r[e + 0]) * inv, __uint_as_float(r[e + 1]) * inv);
            w.y = pack16x2<BF16>(__uint_as_float(r[e + 2]) * inv, __uint_as_float(r[e + 3]) * inv);
            w.z = pack16x2<BF16>(__uint_as_float(r[e + 4]) * inv, __uint_as_float(r[e + 5]) * inv);
            w.w = pack16x2<BF16>(__uint_as_float(r[e + 6]) * inv, __uint_as_float(r[e + 7]) * inv);
            dst[j] = w;
          }
        }
      } else {
#pragma unroll
      for (int p = 0; p < kOutPanels; ++p) {
        if (row == 0) tma_store_wait_read();  // the store that used the buffer last has read it
        named_barrier_sync(1 + x, kBM);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int e = p * 64 + 8 * j;
          uint4 w;
          w.x = pack16x2<BF16>(__uint_as_float(r[e + 0]) * inv, __uint_as_float(r[e + 1]) * inv);
          w.y = pack16x2<BF16>(__uint_as_float(r[e + 2]) * inv, __uint_as_float(r[e + 3]) * inv);
          w.z = pack16x2<BF16>(__uint_as_float(r[e + 4]) * inv, __uint_as_float(r[e + 5]) * inv);
          w.w = pack16x2<BF16>(__uint_as_float(r[e + 6]) * inv, __uint_as_float(r[e + 7]) * inv);
          *reinterpret_cast<uint4*>(stage + ((j ^ (row & 7)) << 4)) = w;
        }
        fence_proxy_async();  // the store reads shared memory through the async proxy
        named_barrier_sync(1 + x, kBM);
        if (row == 0) {
          tma_store_4d(&tm_o, sm.o_stage[x], p * 64, it.row0 + it.q0 - a.q_start + x * kBM, it.h, PACKED ? 0 : it.b);
          tma_store_commit();
        }
      }
      }
      if (qi < (PACKED ? it.len : T) && lse_row) *lse_row = valid ? m_used + log2f(l) : 0.f;
      KB_FACC(6);
    }
    if (row == 0) tma_store_wait_all();
#ifdef KB_TRACE_FWD
    if (blockIdx.x == 60 && threadIdx.x == 0)
      for (int i = 0; i < 8; ++i) g_fwtrace[16 + i] = acc_t[i];
#endif
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    if (sm.abort_flag) __nanosleep(1000000);  // let copies still in flight land before the CTA goes away
    tmem_dealloc(tmem, kTmemCols);
  }
}

// `f8`: the scales of 8-bit inputs (FP8 only; q, k, v of `p` are then e4m3 tensors with byte strides)
template <int D, bool BF16, bool PACKED, bool FP8>
int launch(const kb_sa_fwd_params& p, int32_t c, int32_t back, cudaStream_t s, const kb_sa_fwd_fp8_params* f8 = nullptr) {
  CUtensorMap tm_q, tm_k, tm_v, tm_o;
  const int32_t H_kv = p.H_kv > 0 ? p.H_kv : p.H;
  const int32_t Tq = p.T - p.q_start;  // rows of q, o and lse
  // a packed batch is ONE batch entry of `total_rows` rows as far as the maps go
  const int32_t mapB = p.cu_seqlens ? 1 : p.B, mapTq = p.cu_seqlens ? p.total_rows : Tq, mapT = p.cu_seqlens ? p.total_rows : p.T;
  const bool maps_ok =
      FP8 ? make_tile_map_4d_u8(&tm_q, p.q, mapB, p.H, mapTq, D, kBM) && make_tile_map_4d_u8(&tm_k, p.k, mapB, H_kv, mapT, D, kBN) &&
                make_tile_map_4d_u8(&tm_v, p.v, mapB, H_kv, mapT, D, kBN)
          : make_tile_map_4d(&tm_q, p.q, mapB, p.H, mapTq, D, kBM) && make_tile_map_4d(&tm_k, p.k, mapB, H_kv, mapT, D, kBN) &&
                make_tile_map_4d(&tm_v, p.v, mapB, H_kv, mapT, D, kBN);
  if (!maps_ok || !make_tile_map_4d(&tm_o, out_view(p.o, p.o_stride, p.H, mapTq, D), mapB, p.H, mapTq, D, kBM))
    return KB_ERR_UNSUPPORTED;
  // chunk lengths that are multiples of the work item's rows get the instance with the straight-line schedule
  const bool fast = c % (kBM * kQTiles) == 0;
  auto kern = fast ? sa_fwd_sm100_kernel<D, BF16, PACKED, FP8, true> : sa_fwd_sm100_kernel<D, BF16, PACKED, FP8, false>;
  constexpr size_t smem = sizeof(FwdSmem<D>);
  static_assert(sizeof(FwdSmem<D>) <= 232448, "forward shared memory exceeds the 227 KB a CTA may have");
  int dev = 0, n_sm = 0;
  if (!device_sm_count(&dev, &n_sm)) return KB_ERR_LAUNCH;
  static std::atomic<bool> smem_opted_in[kMaxDevices], smem_opted_in_fast[kMaxDevices];
  KB_CUDA_TRY(opt_in_smem_once(kern, smem, dev, fast ? smem_opted_in_fast : smem_opted_in));
  FwdArgs a;
  a.o = p.o;
  a.lse = p.lse;
  a.lens = p.lens;
  a.lens_stride = p.lens_stride;
  {
    const kb_tensor4 ov = out_view(p.o, p.o_stride, p.H, mapTq, D);
    a.o_sb = ov.stride[0], a.o_sh = ov.stride[1], a.o_st = ov.stride[2];
    const bool lse_packed = p.lse_stride[0] == 0 && p.lse_stride[1] == 0;
    a.lse_sb = lse_packed ? (int64_t)p.H * mapTq : p.lse_stride[0];
    a.lse_sh = lse_packed ? (int64_t)mapTq : p.lse_stride[1];
    if (p.cu_seqlens) a.o_sb = a.lse_sb = 0;  // the sequence's first row carries the batch offset
  }
  a.B = p.B;
  a.H = p.H;
  a.T = p.T;
  a.c = c;
  a.back = back;
  a.q_start = p.q_start;
  a.cu = p.cu_seqlens;
  a.fd_qblocks = kb_fastdiv_make(kb_cdiv_i32(Tq, kBM * kQTiles));
  a.fd_H = kb_fastdiv_make(p.H);
  a.fd_c = kb_fastdiv_make(c);
  a.fd_group = kb_fastdiv_make(p.H / H_kv);
  a.scale_log2 = p.sm_scale * kLog2e;
  a.status = p.status;
  a.q_scale = f8 ? f8->q_scale : nullptr;
  a.k_scale = f8 ? f8->k_scale : nullptr;
  a.v_scale = f8 ? f8->v_scale : nullptr;
  a.v_scale_max = f8 ? f8->v_scale_max : nullptr;
  a.n128 = kb_cdiv_i32(p.T, 128);
  a.Hk = H_kv;
  const int64_t n_items = (int64_t)p.B * p.H * kb_cdiv_i32(Tq, kBM * kQTiles);
  if (n_items > (int64_t)1 << 30) return KB_ERR_TOO_LARGE;
  const unsigned grid = (unsigned)(n_items < n_sm ? n_items : n_sm);  // persistent: one CTA per SM
  kern<<<grid, kThreads, smem, s>>>(tm_q, tm_k, tm_v, tm_o, a);
  KB_LAUNCH_CHECK("sa_fwd_sm100_kernel");
  return KB_OK;
}

}  // namespace

int sa_fwd_sm100(const kb_sa_fwd_params& p, int32_t c, int32_t back, cudaStream_t s) {
  if (!(p.sm_scale > 0.f) || reinterpret_cast<uintptr_t>(p.o) % 16) return KB_ERR_UNSUPPORTED;
  const bool bf16 = p.dtype == KB_BF16;
  if (p.cu_seqlens) {
    if (p.D == 64) return bf16 ? launch<64, true, true, false>(p, c, back, s) : launch<64, false, true, false>(p, c, back, s);
    if (p.D == 128) return bf16 ? launch<128, true, true, false>(p, c, back, s) : launch<128, false, true, false>(p, c, back, s);
    return KB_ERR_UNSUPPORTED;
  }
  if (p.D == 64) return bf16 ? launch<64, true, false, false>(p, c, back, s) : launch<64, false, false, false>(p, c, back, s);
  if (p.D == 128) return bf16 ? launch<128, true, false, false>(p, c, back, s) : launch<128, false, false, false>(p, c, back, s);
  return KB_ERR_UNSUPPORTED;
}

// 8-bit (e4m3) q, k, v with per-tile scales; head dim 128, padded layout, all query rows.
int sa_fwd_sm100_fp8(const kb_sa_fwd_fp8_params& f, int32_t c, int32_t back, cudaStream_t s) {
  if (!(f.sm_scale > 0.f) || reinterpret_cast<uintptr_t>(f.o) % 16 || f.D != 128) return KB_ERR_UNSUPPORTED;
  kb_sa_fwd_params p = {};
  p.q = f.q, p.k = f.k, p.v = f.v;
  p.o = f.o, p.lse = f.lse;
  p.lens = f.lens, p.lens_stride = f.lens_stride;
  p.B = f.B, p.H = f.H, p.T = f.T, p.D = f.D, p.H_kv = f.H_kv;
  p.dtype = f.out_dtype;
  p.context_size = f.context_size, p.back_contexts = f.back_contexts;
  p.sm_scale = f.sm_scale, p.flags = f.flags, p.status = f.status;
  return f.out_dtype == KB_BF16 ? launch<128, true, false, true>(p, c, back, s, &f) : launch<128, false, false, true>(p, c, back, s, &f);
}

}  // namespace kb

#ifdef KB_TRACE_FWD
extern "C" __attribute__((visibility("default"))) int kb_debug_trace_fwd(long long* out) {
  return (int)cudaMemcpyFromSymbol(out, kb::g_fwtrace, sizeof(kb::g_fwtrace));
}
#endif
