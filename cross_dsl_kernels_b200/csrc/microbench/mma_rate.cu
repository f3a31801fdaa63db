// Micro-benchmark (stand-alone program, not part of the library): how fast does a warp get tcgen05.mma instructions
// out (A in tensor memory, B in shared memory, M = 128, small N), and does it depend on how accumulators are shared
// between consecutive MMAs and between issuing warps?  One CTA; every wait is time-bounded.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_rate mma_rate.cu && ./mma_rate
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include "../umma.cuh"
using namespace xdk;

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e_), __LINE__); return 1; } } while (0)

struct Res { long long cycles; long long ns; };

// mode: warps = issuing warps; accs = accumulators each warp rotates over; shared_acc = 1: all warps use the same set
template <int KIND>  // 0: f16 (K=16), 2: tf32 (K=8)
__global__ void __launch_bounds__(256, 1) mma_kernel(int warps, int accs, int shared_acc, int n, int reps, int a_rot, Res* out) {
  __shared__ __align__(1024) unsigned char bsm[32768];
  __shared__ uint64_t done_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ long long t_begin[8], t_end[8], c_begin[8], c_end[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 32768 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(bsm)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(&done_bar, warps); mbar_fence_init(); }
  if (warp == 7) tmem_alloc<512>(&tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  // zero the A region and accumulators so no NaN slow paths (if any) matter
  if (warp < 4) {
    uint32_t z[16];
    for (int i = 0; i < 16; ++i) z[i] = 0;
    for (int c = 0; c < 512; c += 16) tmem_st16(tmem + ((uint32_t)(warp * 32) << 16) + c, z);
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp < warps && lane == 0) {
    const uint64_t bdesc = umma_desc(smem_u32(bsm), 128, 1024);
    const uint32_t idesc = umma_idesc(n, KIND);
    const int per_warp_cols = (256 / warps) & ~31;  // accumulator columns per warp
    c_begin[warp] = clock64(); t_begin[warp] = (long long)global_timer_ns();
    for (int r = 0; r < reps; ++r) {
      const int sel = r % accs;
      const uint32_t acc = tmem + (shared_acc ? 0 : warp * per_warp_cols) + sel * n;
      const uint32_t a = tmem + 256 + ((r % a_rot) * 8) + (warp * 32 % 224);
      if (KIND == 0) umma_f16_ta(acc, a, bdesc, idesc, r >= accs);
      else umma_tf32_ta(acc, a, bdesc, idesc, r >= accs);
    }
    c_end[warp] = clock64();  // issue done
    umma_commit(&done_bar);
  }
  if (threadIdx.x == 0) {
    mbar_wait(&done_bar, 0);
    const long long t1 = (long long)global_timer_ns();
    long long cb = c_begin[0], ce = c_end[0], tb = t_begin[0];
    for (int w = 1; w < warps; ++w) { if (c_end[w] - c_begin[w] > ce - cb) { cb = c_begin[w]; ce = c_end[w]; } if (t_begin[w] < tb) tb = t_begin[w]; }
    out->cycles = ce - cb;
    out->ns = t1 - tb;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 7) { tc_fence_after(); tmem_dealloc<512>(tmem); }
}

int main() {
  Res* d; CK(cudaMalloc(&d, sizeof(Res)));
  const int reps = 2048;
  struct Case { const char* name; int kind, warps, accs, shared, n, a_rot; };
  const Case cases[] = {
      {"tf32 N16 1 warp, same acc", 2, 1, 1, 0, 16, 1}, {"tf32 N16 1 warp, 2 accs alternating", 2, 1, 2, 0, 16, 1}, {"tf32 N16 1 warp, 4 accs", 2, 1, 4, 0, 16, 1},
      {"tf32 N16 1 warp, 8 accs", 2, 1, 8, 0, 16, 1}, {"tf32 N16 1 warp, 16 accs", 2, 1, 16, 0, 16, 1},
      {"tf32 N32 1 warp, same acc", 2, 1, 1, 0, 32, 1}, {"tf32 N32 1 warp, 2 accs", 2, 1, 2, 0, 32, 1}, {"tf32 N32 1 warp, 8 accs", 2, 1, 8, 0, 32, 1},
      {"tf32 N64 1 warp, same acc", 2, 1, 1, 0, 64, 1}, {"tf32 N64 1 warp, 4 accs", 2, 1, 4, 0, 64, 1}, {"tf32 N32 1 warp, 4 accs", 2, 1, 4, 0, 32, 1},
      {"tf32 N16 4 warps, own acc each", 2, 4, 1, 0, 16, 1}, {"tf32 N16 4 warps, 2 accs each", 2, 4, 2, 0, 16, 1}, {"tf32 N16 4 warps, 4 accs each", 2, 4, 4, 0, 16, 1},
      {"tf32 N16 4 warps, all same acc", 2, 4, 1, 1, 16, 1},
      {"tf32 N32 4 warps, own acc each", 2, 4, 1, 0, 32, 1}, {"tf32 N32 4 warps, 2 accs each", 2, 4, 2, 0, 32, 1},
      {"tf32 N16 8 warps, own acc each", 2, 7, 1, 0, 16, 1}, {"tf32 N16 2 warps, own acc each", 2, 2, 1, 0, 16, 1},
      {"tf32 N16 1 warp, same acc, A rotates 8", 2, 1, 1, 0, 16, 8}, {"tf32 N16 1 warp, 8 accs, A rotates 8", 2, 1, 8, 0, 16, 8},
      {"f16 N16 1 warp, same acc", 0, 1, 1, 0, 16, 1}, {"f16 N16 1 warp, 4 accs", 0, 1, 4, 0, 16, 1}, {"f16 N16 4 warps, own acc each", 0, 4, 1, 0, 16, 1},
      {"f16 N64 1 warp, same acc", 0, 1, 1, 0, 64, 1}, {"f16 N64 4 warps, own acc", 0, 4, 1, 0, 64, 1},
  };
  for (const Case& c : cases) {
    Res best = {1LL << 60, 1LL << 60};
    for (int it = 0; it < 4; ++it) {
      if (c.kind == 0) mma_kernel<0><<<1, 256>>>(c.warps, c.accs, c.shared, c.n, reps, c.a_rot, d);
      else mma_kernel<2><<<1, 256>>>(c.warps, c.accs, c.shared, c.n, reps, c.a_rot, d);
      CK(cudaDeviceSynchronize());
      Res r; CK(cudaMemcpy(&r, d, sizeof(r), cudaMemcpyDeviceToHost));
      if (r.ns < best.ns) best = r;
    }
    const double total = (double)reps * c.warps;
    printf("%-44s issue %7.1f cycles/MMA/warp   complete %7.1f ns/MMA aggregate (%6.1f cycles at 1.965 GHz)\n", c.name,
           (double)best.cycles / reps, best.ns / total, best.ns / total * 1.965);
    fflush(stdout);
  }
  return 0;
}
