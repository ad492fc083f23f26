// The committed sm_100a tile table: tile shapes and pipeline depths of every kernel family, in one
// place.  The kernels take their constants from here and kb_sa_tile_config() reports the same
// numbers, so the table a caller reads cannot drift from what the GPU runs.  It replaces the
// reference's per-GPU config tables and autotune search (src/streaming_attention/kernel.py:17-192,
// 1133-1267); the measurements behind the choices are summarised under profiles/.
#pragma once

namespace kb {
namespace tiles {

// tcgen05 forward (f16 / bf16, D 64 or 128): a work item is kFwdQTiles tiles of kFwdQRows query rows
// that share every K/V tile of kFwdKeys keys; K and V rings.
constexpr int kFwdQRows = 128, kFwdQTiles = 2, kFwdKeys = 128;
constexpr int kFwdStagesK = 2, kFwdStagesV = 2;

// tcgen05 backward, two passes: kTwoPassStationary rows stay in shared memory, tiles of
// kTwoPassStreamed rows stream past them through two rings (first / second streamed operand).
constexpr int kTwoPassStationary = 128, kTwoPassStreamed = 128;
constexpr int kTwoPassStagesFirst = 3, kTwoPassStagesSecond = 2;

// tcgen05 backward, scores evaluated once.  Main kernel: a key tile stays, query tiles stream (Q ring;
// dO single buffered; K double buffered across items).  dQ kernel: a query tile's accumulator stays,
// (dS, K) tile pairs stream.
constexpr int kMainKeys = 128, kMainQueries = 128, kMainStagesQ = 2, kMainStagesK = 2;
constexpr int kDqQueries = 128, kDqKeys = 128, kDqStages = 3;

// generic CUDA-core kernels: square tiles, no software pipeline
constexpr int generic_tile(int D) { return D <= 128 ? 64 : 32; }
constexpr int kGenericStages = 1;

}  // namespace tiles
}  // namespace kb
