// kb_sa_bwd_noalloc: the streaming-attention backward for callers that cannot hand the
// library a scratch buffer.
//
// The regular backward (kb_sa_bwd) needs B*H*T floats of scratch for delta = rowsum(O * dO),
// which the dQ pass writes and the dK/dV pass reads; its caller allocates them.  Some hosts
// cannot do that: an inference-runtime plugin whose execute hook receives only its input and
// output bindings and is forbidden to allocate, a service that reserved the whole device
// memory for its own arena at start-up (a later cudaMalloc simply fails), or a latency-bound
// loop that cannot afford the device-wide synchronisation a cudaMalloc / cudaFree pair implies.
// For them this file keeps the scratch in a fixed array inside the library image.
//
// Properties a caller must know:
//   * the array holds KB_NOALLOC_MAX_ROWS floats (8 MiB) on every GPU that uses the library,
//     until the process exits; a problem with B*H*T above that is refused with
//     KB_ERR_TOO_LARGE and nothing is launched;
//   * the first call on each device looks up the array's device address (one
//     cudaGetSymbolAddress with that device current).  With the CUDA runtime's lazy module
//     loading that is also the moment the device sets the 8 MiB aside, so make that first call
//     during set-up: before any stream capture is started on that device, and before the host
//     hands the rest of the device memory to an arena of its own;
//   * it runs the two-pass kernels as they are: one key/value head per query head and contiguous
//     dq / dk / dv only (H_kv other than 0 or H, or any *_stride set, returns
//     KB_ERR_UNSUPPORTED with nothing launched), and none of the KB_FLAG_BWD_SKIP_* timing flags
//     (a pass that is skipped would leave the other reading an EARLIER call's delta out of the
//     shared array; KB_ERR_BAD_ARGUMENT);
//   * every call on a device shares the one array and it keeps the previous call's values.
//     Nothing in it has to start at zero: the dQ pass overwrites every entry the dK/dV pass of
//     the same call reads.  Two calls that overlap on the same GPU (different streams) race on
//     it, so serialise them;
//   * no cudaMalloc, cudaFree or allocating library routine is called, here or below.
#include <mutex>

#include "common.cuh"

namespace {

static __device__ __align__(256) float g_delta_scratch[KB_NOALLOC_MAX_ROWS];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
float* g_scratch_addr[kMaxDevices] = {};  // per device: address of that device's copy of the array

// In host code `g_delta_scratch` is only a handle for the runtime, not a device address, so the
// address each device gives the array is looked up once, with that device current.
int scratch_for_current_device(float** out) {
  int dev = -1;
  KB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return KB_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_scratch_addr[dev]) {
    float* ptr = nullptr;
    KB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_delta_scratch));
    if (!ptr) return KB_ERR_LAUNCH;
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return KB_OK;
}

}  // namespace

extern "C" int kb_sa_bwd_noalloc(const kb_sa_bwd_params* p, void* stream) {
  if (!p) return KB_ERR_BAD_ARGUMENT;
  if (p->B < 0 || p->H < 0 || p->T < 0) return KB_ERR_BAD_ARGUMENT;
  // every call must write the delta it reads: no partial backward out of the shared array
  if (p->flags & (KB_FLAG_BWD_SKIP_DQ | KB_FLAG_BWD_SKIP_DKDV | KB_FLAG_BWD_SKIP_DELTA)) return KB_ERR_BAD_ARGUMENT;
  const int64_t rows = (int64_t)p->B * p->H * p->T;
  if (rows > (int64_t)KB_NOALLOC_MAX_ROWS) return KB_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != KB_OK) return rc;
  kb_sa_bwd_params q = *p;
  q.delta_ws = scratch;  // whatever the caller put there is ignored
  q.ds_ws = nullptr;  // the two-pass kernels need no scratch besides delta
  q.ds_ws_bytes = 0;
  return kb_sa_bwd(&q, stream);
}
