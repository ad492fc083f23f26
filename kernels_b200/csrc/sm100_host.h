// Host helper for the sm_100a kernels: TMA tensor maps over strided [B, H, T, D] tensors and the
// per-device state a launch needs (SM count, the kernels' shared-memory opt-in), looked up once.
// The driver's encoder is looked up at run time, so the library carries no link-time
// dependency on libcuda and still loads on a machine without a GPU driver.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <atomic>

#include "../../include/kernels_b200.h"

namespace kb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

constexpr int kMaxDevices = 64;

// Current device and its SM count; the attribute query is made once per device.
inline bool device_sm_count(int* dev_out, int* n_sm_out) {
  static std::atomic<int> cache[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  int n = (dev >= 0 && dev < kMaxDevices) ? cache[dev].load(std::memory_order_relaxed) : 0;
  if (n <= 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return false;
    if (dev >= 0 && dev < kMaxDevices) cache[dev].store(n, std::memory_order_relaxed);
  }
  *dev_out = dev;
  *n_sm_out = n;
  return true;
}

// Opt a kernel in to `bytes` of dynamic shared memory once per device (the attribute belongs to the
// device's copy of the function).  `done` is the caller's static per-kernel table.
template <typename Kern>
inline cudaError_t opt_in_smem_once(Kern kern, size_t bytes, int dev, std::atomic<bool> (&done)[kMaxDevices]) {
  if (dev >= 0 && dev < kMaxDevices && done[dev].load(std::memory_order_acquire)) return cudaSuccess;
  const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess && dev >= 0 && dev < kMaxDevices) done[dev].store(true, std::memory_order_release);
  return e;
}

// What a tensor map over a [B, H, T, D] tensor depends on; maps are cached by it per host thread (a
// training loop calls with the same tensors' addresses step after step, and encoding the four to seven
// maps of a launch costs more host time than the launch itself).  A map holds only the address and the
// layout, never data, so a stale entry for memory that was freed and reallocated with the same layout
// is still the right map.
struct TileMapKey {
  const void* data;
  int64_t stride[3];
  int32_t B, H, T, D, box_rows;
};
struct TileMapCache {
  static constexpr int kEntries = 32;
  TileMapKey key[kEntries];
  CUtensorMap map[kEntries];
  bool used[kEntries] = {};
  int next = 0;
};

inline bool encode_tile_map_4d(CUtensorMap* out, const kb_tensor4& t, int B, int H, int T, int D, int box_rows);

// Map over a 16-bit [B, H, T, D] tensor with element strides; a box is [box_rows x 64]
// elements of one (b, h) (128 bytes per row, SWIZZLE_128B); rows past T read as zeros.
// Returns false when the layout cannot be described (the caller then uses the generic path).
inline bool make_tile_map_4d(CUtensorMap* out, const kb_tensor4& t, int B, int H, int T, int D, int box_rows) {
  static thread_local TileMapCache cache;
  TileMapKey k;
  memset(&k, 0, sizeof(k));
  k.data = t.data;
  k.stride[0] = t.stride[0], k.stride[1] = t.stride[1], k.stride[2] = t.stride[2];
  k.B = B, k.H = H, k.T = T, k.D = D, k.box_rows = box_rows;
  if (t.stride[3] == 1) {
    for (int i = 0; i < TileMapCache::kEntries; ++i)
      if (cache.used[i] && memcmp(&cache.key[i], &k, sizeof(k)) == 0) {
        *out = cache.map[i];
        return true;
      }
  }
  if (!encode_tile_map_4d(out, t, B, H, T, D, box_rows)) return false;
  const int slot = cache.next;
  cache.next = (slot + 1) % TileMapCache::kEntries;
  cache.key[slot] = k;
  cache.map[slot] = *out;
  cache.used[slot] = true;
  return true;
}

inline bool encode_tile_map_4d(CUtensorMap* out, const kb_tensor4& t, int B, int H, int T, int D, int box_rows) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return false;
  if (t.stride[3] != 1 || reinterpret_cast<uintptr_t>(t.data) % 16) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
  int64_t st[3] = {t.stride[2], t.stride[1], t.stride[0]};  // t, h, b
  const int64_t extent[3] = {T, H, B};
  // a dimension of extent 1 may carry any stride: give it a harmless valid one
  int64_t fallback = D;
  for (int i = 0; i < 3; ++i) {
    if (extent[i] == 1) st[i] = fallback;
    if (st[i] <= 0 || (st[i] * 2) % 16 || st[i] * 2 >= ((int64_t)1 << 40)) return false;
    fallback = st[i] * extent[i];
  }
  const cuuint64_t strides[3] = {(cuuint64_t)st[0] * 2, (cuuint64_t)st[1] * 2, (cuuint64_t)st[2] * 2};
  const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(t.data), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Map over an 8-bit [B, H, T, D] tensor with element (= byte) strides, D = 128: a box is [box_rows x 128] bytes of
// one (b, h) (one 128-byte swizzled line per row); rows past T read as zeros.  Not cached (the 8-bit entry
// point makes three per call).
inline bool make_tile_map_4d_u8(CUtensorMap* out, const kb_tensor4& t, int B, int H, int T, int D, int box_rows) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc || D != 128) return false;
  if (t.stride[3] != 1 || reinterpret_cast<uintptr_t>(t.data) % 16) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
  int64_t st[3] = {t.stride[2], t.stride[1], t.stride[0]};  // t, h, b
  const int64_t extent[3] = {T, H, B};
  int64_t fallback = D;
  for (int i = 0; i < 3; ++i) {
    if (extent[i] == 1) st[i] = fallback;
    if (st[i] <= 0 || st[i] % 16 || st[i] >= ((int64_t)1 << 40)) return false;
    fallback = st[i] * extent[i];
  }
  const cuuint64_t strides[3] = {(cuuint64_t)st[0], (cuuint64_t)st[1], (cuuint64_t)st[2]};
  const cuuint32_t box[4] = {128, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(t.data), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// An output tensor as a strided view: `stride` holds the element strides of its b, h, t axes, all zeros
// meaning [B, H, T, D] contiguous.
inline kb_tensor4 out_view(void* data, const int64_t (&stride)[3], int H, int T, int D) {
  kb_tensor4 t;
  t.data = data;
  const bool packed = stride[0] == 0 && stride[1] == 0 && stride[2] == 0;
  t.stride[0] = packed ? (int64_t)H * T * D : stride[0];
  t.stride[1] = packed ? (int64_t)T * D : stride[1];
  t.stride[2] = packed ? (int64_t)D : stride[2];
  t.stride[3] = 1;
  return t;
}

// Map over a contiguous 16-bit [B, H, T, D] output tensor (same boxes as the inputs).
inline bool make_tile_map_4d_contiguous(CUtensorMap* out, void* data, int B, int H, int T, int D, int box_rows) {
  kb_tensor4 t;
  t.data = data;
  t.stride[3] = 1;
  t.stride[2] = D;
  t.stride[1] = (int64_t)T * D;
  t.stride[0] = (int64_t)H * T * D;
  return make_tile_map_4d(out, t, B, H, T, D, box_rows);
}

}  // namespace kb
