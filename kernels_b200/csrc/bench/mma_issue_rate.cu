// Microbenchmark behind the tile table: SM clocks per tcgen05.mma instruction (M = 128, K = 16, bf16 in,
// fp32 out) when one thread of every SM issues them back to back, for A from shared memory (SS) or TMEM
// (TS), N = 64 / 128 / 256, one accumulator or several in rotation, with and without other warps loading
// TMEM, computing exponentials and reading / writing shared memory.  Operands are whatever the memory
// holds: only timing is measured.  Stand-alone (no torch); every wait is bounded.
// Build and run:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I include -I kernels_b200/csrc -o mma_issue_rate kernels_b200/csrc/bench/mma_issue_rate.cu
#include <cstdio>
#include <cstdlib>
#include "../../../include/kernels_b200.h"
#include "../sm100_ptx.cuh"
using namespace kb::sm100;

// mode bits: 1 = TS (A from TMEM) else SS; 2 = N256 (else N128); 4 = noise: 8 warps tcgen05.ld; 8 = noise: 8 warps ex2/fma loops;
// 16 = noise: 8 warps st.shared; 32 = noise: 8 warps ld.shared broadcast; 64 = N64; 128 = commit after every 8 instrs + wait (dependency)
__global__ void __launch_bounds__(320, 1) k(int mode, int iters, long long* out) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base;
  __shared__ volatile int stop;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); stop = 0; fence_mbar_init(); }
  if (warp == 9) tmem_alloc(&tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base;
  const int N = (mode & 2) ? 256 : ((mode & 64) ? 64 : 128);
  if (warp == 9) {
    if (lane == 0) {
      const uint32_t idesc_ss = make_idesc(true, 128, N, false, false);
      const uint32_t idesc_ts = make_idesc(true, 128, N, false, true);
      const uint32_t a_addr = smem_u32(smem), b_addr = smem_u32(smem + 65536);
      long long t0 = clock64();
      int ph = 0;
      for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          const uint32_t dcol = (mode & 256) ? ((kk & 1) ? 384u : 256u) : ((mode & 512) ? (uint32_t)((kk & 3) * 128) : 256u);
          if (mode & 1)
            mma_ts(tmem + dcol, tmem + (kk / 4) * 64 + (kk % 4) * 8, desc_mnmajor(b_addr + kk * 2048, 16384), idesc_ts, true);
          else
            mma_ss(tmem + dcol, desc_kmajor(a_addr + off), desc_kmajor(b_addr + off), idesc_ss, true);
        }
        if (mode & 128) {
          mma_commit(&bar);
          for (int spin = 0; spin < (1 << 22) && !mbar_try_wait(&bar, ph); ++spin) {}
          ph ^= 1;
        }
      }
      long long t1 = clock64();
      mma_commit(&bar);
      for (int spin = 0; spin < (1 << 24) && !mbar_try_wait(&bar, (mode & 128) ? ph : 0); ++spin) {}
      long long t2 = clock64();
      out[0] = t1 - t0;
      out[1] = t2 - t0;
      stop = 1;
    }
  } else if (warp < 8) {
    const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    float acc = 0.f;
    uint32_t r[32];
    for (int i = 0; i < 32; ++i) r[i] = i + lane;
    for (int round = 0; round < (1 << 22) && !stop; ++round) {
      if (mode & 4) {
        tmem_ld32(t_lane + (warp >> 2) * 64, r);
        tmem_wait_ld();
        acc += __uint_as_float(r[5]);
      }
      if (mode & 8) {
#pragma unroll
        for (int i = 0; i < 32; ++i) acc += ex2_approx(fmaf(__uint_as_float(r[i]), 1.0001f, acc));
      }
      if (mode & 16) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          *reinterpret_cast<uint4*>(smem + 131072 + (warp * 32 + lane) * 128 + ((i ^ (lane & 7)) << 4)) = make_uint4(r[0], r[1], r[2], r[3]);
      }
      if (mode & 32) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float4 v;
          asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(smem_u32(smem + 131072 + 65536 + i * 16 + (warp & 1) * 256)));
          acc += v.x;
        }
      }
      if (!(mode & 60)) __nanosleep(200);
    }
    if (acc == 123.456f) out[7] = 1;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, 512);
}

int main() {
  long long* d;
  cudaMalloc(&d, 64);
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  const int iters = 2000;
  int modes[] = {0, 1, 2, 3, 64, 128, 129, 256, 257, 512, 513, 256 + 64, 512 + 64, 4, 5, 8, 9, 16, 17, 32, 33, 60, 61, 256 + 60, 257 + 60};
  for (int m : modes) {
    for (int rep = 0; rep < 2; ++rep) {
      k<<<148, 320, 200 * 1024>>>(m, iters, d);
      cudaError_t e = cudaDeviceSynchronize();
      if (e != cudaSuccess) { printf("mode %d: %s\n", m, cudaGetErrorString(e)); return 1; }
    }
    long long h[2];
    cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
    printf("mode %3d (%s N%d%s%s%s%s%s%s): issue %.1f clk/instr, complete %.1f clk/instr\n", m, (m & 1) ? "TS" : "SS",
           (m & 2) ? 256 : ((m & 64) ? 64 : 128), (m & 128) ? " dep8" : "", (m & 4) ? " +tmem_ld" : "", (m & 8) ? " +ex2" : "",
           (m & 16) ? " +st.shared" : "", (m & 32) ? " +ld.shared" : "", (m & 256) ? " 2acc" : ((m & 512) ? " 4acc" : ""), h[0] / (8.0 * iters), h[1] / (8.0 * iters));
  }
  return 0;
}
