/*
 * kernels_b200 — C ABI of the B200 (sm_100a) streaming-attention library.
 *
 * The reference project (alexdremov/kernels) has no native boundary: its Python op
 * bodies launch Triton kernels directly.  This header declares the entry points that
 * those op bodies call instead; each one cites the reference interface it replaces
 * (paths are inside the reference project).
 *
 * Conventions
 *   - every pointer is a raw device pointer unless stated otherwise; the library never
 *     allocates or frees memory the caller can see and keeps no pointer after returning;
 *   - tensors are [B, H, T, D]; inputs carry explicit ELEMENT strides, outputs are
 *     contiguous;
 *   - all launches go to the `stream` argument (a cudaStream_t passed as void*) on the
 *     device that is current for the calling thread;
 *   - return value 0 = success, otherwise a kb_status code; kb_strerror() names it;
 *   - `status` (optional) points at KB_STATUS_WORDS int32 words the kernels can write
 *     from the device (pinned host memory is fine).  Word 0 becomes non-zero when a
 *     bounded wait inside a kernel gave up; the caller reads it after synchronising.
 */
#ifndef KERNELS_B200_H_
#define KERNELS_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define KB_API __attribute__((visibility("default")))
#else
#define KB_API
#endif

#define KB_STATUS_WORDS 4

typedef enum kb_status {
  KB_OK = 0,
  KB_ERR_BAD_ARGUMENT = 1,   /* null pointer, negative size, context_size < 1, ...            */
  KB_ERR_UNSUPPORTED = 2,    /* dtype / head_dim / stride combination no kernel covers       */
  KB_ERR_LAUNCH = 3,         /* the CUDA runtime refused the launch (see kb_last_cuda_error) */
  KB_ERR_DEVICE_TIMEOUT = 4, /* a bounded device-side wait gave up (status word set)         */
  KB_ERR_TOO_LARGE = 5       /* problem exceeds a fixed-size internal buffer                 */
} kb_status;

typedef enum kb_dtype { KB_F32 = 0, KB_F16 = 1, KB_BF16 = 2 } kb_dtype;

/* flags for the attention entry points */
#define KB_FLAG_PRESCALE_QK 1u   /* accepted for signature parity; scaling is always done in fp32 */
#define KB_FLAG_ALLOW_TF32 2u    /* precision="tf32": accepted, fp32 inputs still use IEEE fp32    */
#define KB_FLAG_FORCE_GENERIC 4u /* skip the tcgen05 path even where it applies (tests)           */
/* backward only, for per-kernel timing: leave out kernels of the backward.  A kernel that runs
 * reads what an earlier call over the same inputs left in delta_ws / ds_ws.
 *   two-pass kernels:          SKIP_DQ = no dQ pass (which also forms delta), SKIP_DKDV = no dK/dV pass
 *   single-evaluation kernels: SKIP_DELTA = no delta kernel, SKIP_DKDV = no main kernel (dK, dV, dS),
 *                              SKIP_DQ = no dQ kernel */
#define KB_FLAG_BWD_SKIP_DQ 8u
#define KB_FLAG_BWD_SKIP_DKDV 16u
#define KB_FLAG_BWD_SKIP_DELTA 64u
/* backward only: always take the two-pass kernels (dQ pass + dK/dV pass, no scratch besides delta)
 * even when ds_ws is given */
#define KB_FLAG_BWD_TWO_PASS 32u

/* which kernel family an attention call resolves to (see kb_sa_select_path) */
#define KB_PATH_GENERIC 0 /* CUDA-core path: any dtype, head_dim, stride                 */
#define KB_PATH_SM100 1   /* TMA + tcgen05/TMEM path: f16/bf16, D in {64,128}, dense rows */

typedef struct kb_tensor4 {
  const void* data;
  int64_t stride[4]; /* element strides of the b, h, t, d axes */
} kb_tensor4;

/*
 * Streaming attention forward.
 * Replaces the Triton launch in `attention_forward_adapter`
 * (src/streaming_attention/kernel.py:1273-1337, kernel `_streaming_attn_fwd`, lines 205-430).
 * Rows t >= len_b of `o` are written as 0 and of `lse` as 0; `lse` holds the base-2
 * log-sum-exp (kernel.py:407-408) and may be NULL.
 */
typedef struct kb_sa_fwd_params {
  kb_tensor4 q, k, v;
  void* o;             /* [B,H,T,D] contiguous, same dtype as q */
  float* lse;          /* [B,H,T] contiguous fp32, or NULL       */
  const int32_t* lens; /* [B] or NULL (= every length is T)      */
  int64_t lens_stride;
  int32_t B, H, T, D;
  int32_t dtype; /* kb_dtype */
  int32_t context_size;
  int32_t back_contexts;
  float sm_scale;
  uint32_t flags;
  int32_t* status; /* KB_STATUS_WORDS words, or NULL */
  /* Shared key/value heads (grouped-query attention; an extension, the reference requires equal head
   * counts, src/streaming_attention/kernel.py:1291).  0 or H: k and v have H heads.  Otherwise k and v are
   * [B, H_kv, T, D], H a multiple of H_kv, and query head h reads key/value head h / (H / H_kv).  Only the
   * tcgen05 kernels take H_kv != H; other calls return KB_ERR_UNSUPPORTED with nothing launched (the caller
   * then repeats the K/V heads itself). */
  int32_t H_kv;
  /* Output layout (an extension: the reference allocates its outputs itself, kernel.py:1304-1308).  All
   * zeros: `o` is [B,H,T,D] and `lse` [B,H,T], contiguous.  Otherwise the element strides of o's b, h, t
   * axes (d has stride 1; multiples of 8 elements) and of lse's b, h axes (t has stride 1).  Only the
   * tcgen05 kernels take a strided output; other calls return KB_ERR_UNSUPPORTED with nothing launched. */
  int64_t o_stride[3];
  int64_t lse_stride[2];
  /* Streaming step (an extension; the reference has no key/value cache, its mask, kernel.py:1540-1542,
   * defines the result): 0 for the reference's call.  Otherwise only the queries of the positions
   * [q_start, T) are given and computed: q, o and lse have T - q_start rows, row r standing at position
   * q_start + r, while k and v hold all T positions (an inference step: the new chunk of queries against a
   * cache of the last back_contexts + 1 chunks, whose first row must lie on a chunk boundary).  `lens` still
   * counts positions.  Only the tcgen05 kernels take q_start != 0; other calls return KB_ERR_UNSUPPORTED. */
  int32_t q_start;
  /* Packed batch in ONE launch (what kb_sa_fwd_varlen calls; NULL for every other call): DEVICE pointer to
   * B + 1 non-decreasing row offsets.  q, k, v then describe one batch entry of `total_rows` rows (the batch
   * stride is ignored), sequence b owning the rows [cu_seqlens[b], cu_seqlens[b + 1]); o_stride / lse_stride
   * give the h and t strides of the packed outputs; T is the LONGEST sequence; lens must be NULL and q_start 0.
   * tcgen05 kernels only. */
  const int32_t* cu_seqlens;
  int32_t total_rows;
} kb_sa_fwd_params;

KB_API int kb_sa_fwd(const kb_sa_fwd_params* p, void* stream);

/*
 * Streaming attention forward on 8-bit floating-point inputs (e4m3) with per-tile scales; no counterpart in the
 * reference, whose kernels take fp32 / fp16 / bf16 (src/streaming_attention/kernel.py:1288-1295).  Both
 * matmuls run as tcgen05 kind::f8f6f4, which covers 32 reduction elements per instruction instead of 16.
 *   q [B, H, T, D], k, v [B, H_kv, T, D]: e4m3 bytes with element (= byte) strides, unit stride along D, rows
 *     16-byte aligned; D = 128;
 *   q_scale [B, H, n], k_scale, v_scale [B, H_kv, n] with n = ceil(T / 128): the real value of an element is
 *     byte value * scale of its tile of 128 consecutive rows; v_scale_max [B, H_kv] = the largest v_scale of
 *     each key/value head (> 0);
 *   o [B, H, T, D] contiguous in `out_dtype` (KB_F16 or KB_BF16), lse [B, H, T] fp32 base 2 or NULL.
 * The result is the streaming attention of the DEQUANTISED q, k, v up to the rounding of the probabilities to
 * e4m3 (three mantissa bits) before P V: output max-abs <= 5e-2 and relative L2 <= 4e-2 against the fp32
 * reference on the dequantised inputs is the tolerance the tests hold it to.  Forward only.
 */
typedef struct kb_sa_fwd_fp8_params {
  kb_tensor4 q, k, v;
  const float* q_scale;
  const float* k_scale;
  const float* v_scale;
  const float* v_scale_max;
  void* o;
  float* lse;
  const int32_t* lens;
  int64_t lens_stride;
  int32_t B, H, H_kv, T, D;
  int32_t out_dtype;
  int32_t context_size;
  int32_t back_contexts;
  float sm_scale;
  uint32_t flags;
  int32_t* status;
} kb_sa_fwd_fp8_params;

KB_API int kb_sa_fwd_fp8(const kb_sa_fwd_fp8_params* p, void* stream);

/*
 * Streaming attention backward: dQ, dK, dV from (q, k, v, o, lse, do).
 * Replaces both launches in `attention_backward_adapter`
 * (src/streaming_attention/kernel.py:1363-1442: `_streaming_attn_bwd_precompute`, lines
 * 453-514, and `_streaming_attn_bwd`, lines 530-635).
 * Two kernel families serve 16-bit inputs with D in {64, 128}; both are free of atomics and
 * bitwise repeatable:
 *   - single evaluation (taken when `ds_ws` is given and KB_FLAG_BWD_TWO_PASS is not set): a small
 *     kernel forms delta = rowsum(o * do); one persistent kernel walks the transposed schedule
 *     once, produces dK and dV and leaves every 16-bit dS tile in the scratch `ds_ws`; a second
 *     persistent kernel turns the saved tiles into dQ.  Five matmuls per tile pair;
 *   - two passes (`ds_ws` NULL, too small, or KB_FLAG_BWD_TWO_PASS): a dQ pass that also forms delta
 *     and a dK/dV pass, each recomputing the scores: seven matmuls per tile pair, no scratch but
 *     delta.
 * Rows t >= len_b of dq, dk, dv are written as 0.
 */
typedef struct kb_sa_bwd_params {
  kb_tensor4 q, k, v, o, d_o;
  const float* lse; /* [B,H,T] contiguous fp32, base 2 */
  void* dq;         /* [B,H,T,D] contiguous, dtype of q */
  void* dk;
  void* dv;
  float* delta_ws; /* scratch, [B,H,T] fp32, caller-allocated */
  const int32_t* lens;
  int64_t lens_stride;
  int32_t B, H, T, D;
  int32_t dtype;
  int32_t context_size;
  int32_t back_contexts;
  float sm_scale;
  uint32_t flags;
  int32_t* status;
  void* ds_ws;          /* scratch of kb_sa_bwd_workspace_bytes() bytes, 16-byte aligned, or NULL */
  uint64_t ds_ws_bytes; /* its size; too small a scratch selects the two-pass kernels          */
  /* Shared key/value heads, as in kb_sa_fwd_params: k, v, dk, dv are [B, H_kv, T, D]; dk and dv sum the
   * contributions of the H / H_kv query heads of a group (in a fixed order: still bitwise repeatable).
   * Only the single-evaluation tcgen05 kernels take H_kv != H. */
  int32_t H_kv;
  /* Layout of dq, of dk and dv, and of lse, as o_stride / lse_stride of kb_sa_fwd_params (all zeros:
   * contiguous).  Only the single-evaluation tcgen05 kernels take strided gradients. */
  int64_t dq_stride[3];
  int64_t dkv_stride[3];
  int64_t lse_stride[2];
  /* Packed batch in ONE launch per kernel (what kb_sa_bwd_varlen calls; NULL for every other call): DEVICE
   * pointer to B + 1 non-decreasing row offsets, as in kb_sa_fwd_params.  q, k, v, o, d_o then describe one
   * batch entry of `total_rows` rows, dq_stride / dkv_stride / lse_stride give the h and t strides of the packed
   * gradients and of lse ([H, total_rows]), T is the LONGEST sequence, lens must be NULL, delta_ws holds
   * H * total_rows floats and ds_ws kb_sa_bwd_varlen_workspace_bytes() bytes.  Single-evaluation tcgen05
   * kernels only (anything else returns KB_ERR_UNSUPPORTED with nothing launched). */
  const int32_t* cu_seqlens;
  int32_t total_rows;
} kb_sa_bwd_params;

KB_API int kb_sa_bwd(const kb_sa_bwd_params* p, void* stream);

/* Host-only: bytes of `ds_ws` the single-evaluation backward needs for this problem: one 32 KB
 * tile per (key tile, query tile) slot, B * H * ceil(T / 128) * W tiles with W the most query tiles
 * a 128-row key tile meets under (context_size, back_contexts).  0 when no such kernel covers
 * (dtype, D).  The amount grows with (back_contexts + 1) * context_size: a caller that finds it too
 * large passes ds_ws = NULL and gets the two-pass kernels. */
KB_API uint64_t kb_sa_bwd_workspace_bytes(int32_t B, int32_t H, int32_t T, int32_t D, int32_t dtype,
                                          int32_t context_size, int32_t back_contexts);

/*
 * Streaming attention backward without caller-provided scratch.  No counterpart in the
 * reference (its Python op body allocates `delta` itself, kernel.py:1380); it exists for hosts
 * that cannot allocate device memory around the call: a runtime plugin whose execute hook only
 * gets input and output bindings, a process that gave all device memory to its own arena, a
 * latency-bound loop that cannot pay for cudaMalloc's device synchronisation.
 * Same parameter block as kb_sa_bwd; `delta_ws` and `ds_ws` are ignored (the two-pass kernels
 * run, which need no other scratch).  What those kernels do not take, this entry point does not
 * take either: shared key/value heads (H_kv other than 0 or H) and strided gradients (dq_stride,
 * dkv_stride, lse_stride set) return KB_ERR_UNSUPPORTED with nothing launched.  The
 * KB_FLAG_BWD_SKIP_* timing flags are refused (KB_ERR_BAD_ARGUMENT): a skipped pass would leave
 * the other one reading an earlier call's delta.  The B*H*T floats of delta live in
 * a fixed array inside the library (KB_NOALLOC_MAX_ROWS floats = 8 MiB per GPU, held until the
 * process exits); larger problems return KB_ERR_TOO_LARGE and launch nothing.  The first call
 * on a device resolves the array's address and, under the CUDA runtime's lazy module loading, is
 * when the device sets the 8 MiB aside: make it during set-up, before any stream capture on that
 * device and before the host reserves the remaining device memory for itself.  All calls on a
 * device share the array (it need not be cleared: each call
 * overwrites what it reads), so calls that overlap on one GPU race and must be serialised.
 * Calls no cudaMalloc / cudaFree or allocating library routine.
 */
#define KB_NOALLOC_MAX_ROWS (1 << 21)
KB_API int kb_sa_bwd_noalloc(const kb_sa_bwd_params* p, void* stream);

/*
 * Streaming attention over a PACKED batch (no counterpart in the reference, whose callers hold padded
 * [B, T] batches with `lens`, kernel.py:1586-1652): the sequences lie one after the other along the token
 * axis, q / o / dq as [total, H, D], k / v / dk / dv as [total, H_kv, D], lse as [H, total]; sequence b owns
 * the rows [cu_seqlens[b], cu_seqlens[b + 1]).  No padded row is read, computed or written.  Tiles are counted
 * from every sequence's own first row, so the results equal those of the padded call row for row.  With
 * `cu_seqlens_dev` (the offsets in device memory) the forward is ONE launch over all sequences and the backward
 * one launch of each of its three kernels; without it both launch per sequence over strided views (batch 1,
 * T = the sequence's length).  `cu_seqlens` is read on the HOST in every case.
 * tcgen05 kernels only (f16 / bf16, D 64 or 128).  Scratch of the backward: with `cu_seqlens_dev`, `delta_ws`
 * holds H * total floats and `ds_ws` kb_sa_bwd_varlen_workspace_bytes() bytes; without it, `delta_ws` holds
 * H * max_len floats and `ds_ws` kb_sa_bwd_workspace_bytes(1, H, max_len, ...) bytes per lane, reused from
 * sequence to sequence.
 */
typedef struct kb_sa_varlen_params {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse;      /* forward: written (may be NULL); backward: read */
  const void* d_o; /* backward only, [total, H, D] */
  void* dq;
  void* dk;
  void* dv;
  float* delta_ws;
  void* ds_ws;
  uint64_t ds_ws_bytes;
  const int32_t* cu_seqlens; /* host memory, B + 1 non-decreasing entries, cu_seqlens[0] = 0 */
  int32_t B, H, H_kv, D;
  int32_t dtype;
  int32_t context_size;
  int32_t back_contexts;
  float sm_scale;
  uint32_t flags;
  int32_t* status;
  /* The same offsets in DEVICE memory, or NULL.  When given, the forward is ONE launch over all sequences and
   * the backward one launch per kernel (the kernels read a sequence's first row and length from it) instead of
   * launches per sequence (the host copy is still read, for the checks and the longest sequence). */
  const int32_t* cu_seqlens_dev;
  /* Backward without `cu_seqlens_dev` only.  0 or 1: the per-sequence launches follow one another on `stream`.  2 .. 8: they are spread
   * over that many streams of the library's own (made on the first such call on a device), forked from and
   * joined back into `stream`, so that short sequences, each of which fills only a few SMs, run side by side.
   * Every lane needs scratch of its own: `delta_ws` must then hold lanes * H * max_len floats and `ds_ws`
   * lanes times the bytes of one lane. */
  uint32_t lanes;
} kb_sa_varlen_params;

KB_API int kb_sa_fwd_varlen(const kb_sa_varlen_params* p, void* stream);
KB_API int kb_sa_bwd_varlen(const kb_sa_varlen_params* p, void* stream);

/* Host-only: bytes of `ds_ws` the one-launch packed backward needs (kb_sa_bwd_varlen with `cu_seqlens_dev`):
 * one 32 KB tile per (packed key tile, query-tile slot), H * (total_rows / 128 + B + 1) * W tiles with W the
 * most query tiles a key tile of the longest sequence meets.  0 when no such kernel covers (dtype, D). */
KB_API uint64_t kb_sa_bwd_varlen_workspace_bytes(int32_t B, int32_t H, int32_t total_rows, int32_t max_len, int32_t D,
                                                 int32_t dtype, int32_t context_size, int32_t back_contexts);

/*
 * The projections on either side of the attention operator (no counterpart in the reference, whose callers
 * run torch.nn.Linear around it; the seam is its public call, src/streaming_attention/kernel.py:1599-1652,
 * inputs q, k, v [B, H, T, D] and output O).  Hand-written tcgen05 GEMMs that write / read the attention
 * kernels' own layout, so q, k, v and o cross HBM once:
 *
 * kb_qkv_rope_proj:  [q | k | v] = x w^T with rotary position embedding applied to q and k in the epilogue.
 *   x [B, T, E] and w [(H + 2 H_kv) D, E] (rows: the H query heads, then the H_kv key heads, then the H_kv
 *   value heads; the layout of torch.nn.Linear.weight) are contiguous 16-bit; q [B, H, T, D] and k, v
 *   [B, H_kv, T, D] are written contiguous, ready for kb_sa_fwd (H_kv may be smaller than H).  rope_cos /
 *   rope_sin are fp32 tables [D / 2, T] (entry [i, t] = cos / sin of position t times frequency i), or both
 *   NULL for no rotation; element pairs are (d, d + D / 2) of a head ("rotate half").  No bias.
 *   Needs D in {64, 128}, E a multiple of 64, and H and H_kv multiples of 256 / D (a 256-feature tile holds
 *   whole heads of one of q, k, v); anything else returns KB_ERR_UNSUPPORTED with nothing launched.
 *
 * kb_out_proj:  y = concat_heads(o) w^T.  o [B, H, T, D] with element strides (unit stride along D), w
 *   [E_out, H D] and y [B, T, E_out] contiguous; E_out a multiple of 256.
 *
 * Both launch ONE kernel as thread-block clusters of two CTAs (a pair shares each tcgen05.mma over 256 tokens
 * x 256 features), as many pairs as the device holds at once.
 */
typedef struct kb_qkv_proj_params {
  const void* x;
  const void* w;
  void* q;
  void* k;
  void* v;
  const float* rope_cos;
  const float* rope_sin;
  int32_t B, T, E, H, H_kv, D;
  int32_t dtype;   /* KB_F16 or KB_BF16 */
  int32_t* status; /* KB_STATUS_WORDS words, or NULL */
} kb_qkv_proj_params;

typedef struct kb_out_proj_params {
  kb_tensor4 o;
  const void* w;
  void* y;
  int32_t B, T, H, D, E_out;
  int32_t dtype;
  int32_t* status;
} kb_out_proj_params;

KB_API int kb_qkv_rope_proj(const kb_qkv_proj_params* p, void* stream);
KB_API int kb_out_proj(const kb_out_proj_params* p, void* stream);

/*
 * Dense (non-causal) self-attention forward with key padding by `lens`.
 * Replaces the Triton launch in the op body of `alexdremov_flash_attention::forward`
 * (src/self_attention/kernel.py:362-414, kernel `_self_attn_fwd`, lines 125-302).
 * Same parameter block as the streaming forward; context_size/back_contexts are ignored
 * (the dense schedule is the streaming schedule with a single chunk).
 */
KB_API int kb_fa_fwd(const kb_sa_fwd_params* p, void* stream);

/*
 * Row softmax over the last axis of a [rows, cols] fp32/f16/bf16 matrix.
 * Replaces `softmax_kernel` and its launch in `softmax()` (src/softmax/kernel.py:27-91).
 */
typedef struct kb_softmax_params {
  const void* x;
  void* y;
  int64_t rows, cols;
  int64_t x_row_stride; /* elements; inner stride is 1 (kernel.py:41) */
  int64_t y_row_stride;
  int32_t dtype;
} kb_softmax_params;

KB_API int kb_softmax_fwd(const kb_softmax_params* p, void* stream);

/*
 * Host-only: the tile schedule the kernels walk, for one sequence.
 * fwd_ranges[2*i], fwd_ranges[2*i+1] = first / one-past-last KV tile visited by q tile i
 * (src/streaming_attention/kernel.py:243-244, 282-291); bwd_ranges likewise the q tiles
 * visited by KV tile j (kernel.py:1046-1054).  A tile that lies wholly in the padding
 * gets (0, 0).  Either output pointer may be NULL.  Returns the number of q tiles.
 */
KB_API int kb_sa_plan(int32_t T, int32_t seq_len, int32_t context_size, int32_t back_contexts, int32_t tile_q,
               int32_t tile_k, int32_t* fwd_ranges, int32_t* bwd_ranges);

/*
 * Host-only: the committed tile table that replaces the reference's per-GPU config
 * tables and autotuner (src/streaming_attention/kernel.py:17-192, 1133-1267).
 * Writes the kernel family (KB_PATH_*) and its q/kv tile sizes and pipeline depth for
 * the forward (`which` = 0), the two-pass backward's dQ pass (1) and dK/dV pass (2), the
 * single-evaluation backward's main kernel (3) and dQ kernel (4).
 */
KB_API int kb_sa_tile_config(int32_t dtype, int32_t D, int32_t context_size, uint32_t flags, int32_t unit_inner_stride,
                      int32_t which, int32_t* path, int32_t* tile_q, int32_t* tile_k, int32_t* stages);

/*
 * Self-test of the failure path (no counterpart in the reference, which has no device-side waits): launches
 * one small CTA that waits, with a limit of 1 024 polls, on an mbarrier nobody arrives on, through the same
 * bounded wait every tcgen05 kernel of the library uses.  Nothing faults or hangs: the wait gives up, writes
 * {KB_ERR_DEVICE_TIMEOUT, 900, 0} to `status` (KB_STATUS_WORDS int32, device-visible, e.g. pinned host
 * memory) and the kernel returns.  `seen` (3 device-visible int32) receives: whether the short wait reported
 * success (0 expected), whether a second role's long wait on the same barrier did (0 expected: it leaves on the
 * abort flag), and the abort flag (1 expected).  Read both after synchronising the stream.
 */
KB_API int kb_selftest_wait_timeout(int32_t* status, int32_t* seen, void* stream);

/* number of kernels the library launched since it was loaded (all entry points) */
KB_API int64_t kb_launch_count(void);

KB_API const char* kb_strerror(int status);
KB_API const char* kb_last_cuda_error(void);
KB_API const char* kb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* KERNELS_B200_H_ */
