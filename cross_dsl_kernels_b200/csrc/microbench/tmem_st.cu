// Micro-benchmark (stand-alone program, not part of the library): what does a tcgen05.st / tcgen05.ld cost the
// issuing warp, by width and by number of warps?  One CTA.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o tmem_st tmem_st.cu && ./tmem_st
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include "../umma.cuh"
using namespace xdk;
#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e_), __LINE__); return 1; } } while (0)

__device__ __forceinline__ void st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void st8(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}

// mode 0: st x16, wait every `per_wait` stores; 1: st x32; 2: st x8; 3: ld x16
__global__ void __launch_bounds__(512, 1) k(int warps, int mode, int reps, int per_wait, long long* out) {
  __shared__ uint32_t tmem_slot;
  __shared__ long long t0s[16], t1s[16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 15) tmem_alloc<512>(&tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  uint32_t r[32];
  for (int i = 0; i < 32; ++i) r[i] = lane * 7 + i;
  uint32_t r16[16];
  for (int i = 0; i < 16; ++i) r16[i] = lane + i;
  __syncthreads();
  if (warp < warps) {
    const uint32_t base = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (warp >> 2) * 128;  // own lane quarter, own 128 columns
    const long long t0 = (long long)global_timer_ns();
    const long long c0 = clock64();
    for (int i = 0; i < reps; ++i) {
      const uint32_t a = base + (i & 3) * 32;
      if (mode == 0) { tmem_st16(a, r16); }
      else if (mode == 1) { st32(a, r); }
      else if (mode == 2) { st8(a, r); }
      else { uint32_t q[16]; tmem_ld16(a, q); r16[0] ^= q[3]; }
      if (mode != 3 && (i % per_wait) == per_wait - 1) tmem_wait_st();
    }
    if (mode != 3) tmem_wait_st();
    const long long c1 = clock64();
    const long long t1 = (long long)global_timer_ns();
    if (lane == 0) { t0s[warp] = t0; t1s[warp] = t1; out[2 + warp] = c1 - c0; }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    long long a = t0s[0], b = t1s[0];
    for (int w = 1; w < warps; ++w) { if (t0s[w] < a) a = t0s[w]; if (t1s[w] > b) b = t1s[w]; }
    out[0] = b - a; out[1] = r16[0];
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 15) { tc_fence_after(); tmem_dealloc<512>(tmem); }
}

int main() {
  long long* d; CK(cudaMalloc(&d, 32 * sizeof(long long)));
  const int reps = 4096;
  struct Case { const char* name; int warps, mode, per_wait, cols; };
  const Case cases[] = {
      {"st x16, 1 warp, wait/4", 1, 0, 4, 16}, {"st x16, 4 warps (4 quarters), wait/4", 4, 0, 4, 16}, {"st x16, 8 warps, wait/4", 8, 0, 4, 16},
      {"st x16, 12 warps, wait/4", 12, 0, 4, 16}, {"st x16, 8 warps, wait/1", 8, 0, 1, 16}, {"st x16, 8 warps, wait/16", 8, 0, 16, 16},
      {"st x32, 4 warps, wait/4", 4, 1, 4, 32}, {"st x32, 8 warps, wait/4", 8, 1, 4, 32}, {"st x8, 8 warps, wait/4", 8, 2, 4, 8},
      {"ld x16 (+wait each), 4 warps", 4, 3, 1, 16}, {"ld x16 (+wait each), 8 warps", 8, 3, 1, 16},
  };
  for (const Case& c : cases) {
    long long best = 1LL << 60, h[32];
    for (int it = 0; it < 3; ++it) {
      k<<<1, 512>>>(c.warps, c.mode, reps, c.per_wait, d);
      CK(cudaDeviceSynchronize());
      CK(cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost));
      if (h[0] < best) best = h[0];
    }
    const double bytes = (double)reps * c.warps * 32 * c.cols * 4;
    printf("%-40s %8.1f ns per instr per warp  %7.1f cycles  aggregate %7.1f GB/s = %6.1f B/clk\n", c.name, (double)best / reps,
           (double)best / reps * 1.965, bytes / best, bytes / best / 1.965);
    fflush(stdout);
  }
  return 0;
}
