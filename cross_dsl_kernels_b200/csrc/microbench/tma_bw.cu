// Micro-benchmark (stand-alone program, not part of the library): which HBM rate do the TMA access patterns of
// the tensor-core kernels reach when nothing is computed?  148 CTAs, one producer thread issuing box copies into an
// mbarrier ring, one consumer thread that frees a slot as soon as it has landed; every wait is time-bounded.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o tma_bw tma_bw.cu -lcuda && ./tma_bw
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e_), __LINE__); exit(1); } } while (0)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* b, unsigned n) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(n)); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, unsigned bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* b) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory"); }
__device__ __forceinline__ long long gt() { long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ bool mbar_wait(uint64_t* b, unsigned parity) {
  const long long t0 = gt();
  for (;;) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
    if (ok) return true;
    if (gt() - t0 > 20000000LL) return false;  // 20 ms
  }
}
__device__ __forceinline__ void tma2(void* dst, const CUtensorMap* m, int c0, int c1, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)), "l"(m), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma3(void* dst, const CUtensorMap* m, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(dst)), "l"(m), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk1d(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void* src, unsigned bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

__device__ unsigned g_fault;

struct Args {
  int mode;       // 0: KN boxes [64 k][cols]; 1: packed boxes [rows][128 B]; 2: packed 3-D box, 4 chunks; 3: contiguous 1-D bulk
  int steps;      // steps per CTA
  int ring;       // stages
  int stage_bytes;
  int cols;       // mode 0: columns per CTA; mode 1/2: rows per CTA
  int prefetch;   // steps of look-ahead of the L2 prefetch (0 = off)
  const unsigned char* base;
  long long row_bytes;   // pitch of the matrix
  long long cta_bytes;   // mode 3 / prefetch of modes 1, 2: contiguous bytes per CTA
};

__global__ void __launch_bounds__(128, 1) stream_kernel(Args a, const __grid_constant__ CUtensorMap map) {
  extern __shared__ __align__(1024) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)a.ring * a.stage_bytes);
  uint64_t* empty = full + 16;
  if (threadIdx.x == 0) {
    for (int i = 0; i < a.ring; ++i) mbar_init(full + i, 1), mbar_init(empty + i, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int cta = blockIdx.x;
  if (threadIdx.x == 0) {  // producer
    for (int s = 0; s < a.steps; ++s) {
      const int buf = s % a.ring;
      if (s >= a.ring && !mbar_wait(empty + buf, ((s / a.ring) - 1) & 1)) { atomicOr(&g_fault, 1u); break; }
      mbar_expect_tx(full + buf, (unsigned)a.stage_bytes);
      unsigned char* dst = smem + (size_t)buf * a.stage_bytes;
      if (a.mode == 0) tma2(dst, &map, cta * a.cols, s * 64, full + buf);
      else if (a.mode == 1) tma2(dst, &map, (s % 16) * 128, ((s / 16) * gridDim.x + cta) * a.cols, full + buf);
      else if (a.mode == 2) tma3(dst, &map, 0, ((s / 4) * gridDim.x + cta) * a.cols, (s % 4) * 4, full + buf);
      else bulk1d(dst, a.base + (size_t)cta * a.cta_bytes + (size_t)s * a.stage_bytes, (unsigned)a.stage_bytes, full + buf);
    }
  } else if (threadIdx.x == 32) {  // consumer
    for (int s = 0; s < a.steps; ++s) {
      const int buf = s % a.ring;
      if (!mbar_wait(full + buf, (s / a.ring) & 1)) { atomicOr(&g_fault, 2u); break; }
      mbar_arrive(empty + buf);
    }
  } else if (threadIdx.x == 64 && a.prefetch > 0) {  // L2 prefetcher: contiguous chunks, ahead of the boxes
    if (a.mode == 0) {
      // the 64 rows of step s form one contiguous region of 64 * row_bytes; this CTA prefetches its 1/gridDim share
      const long long region = 64LL * a.row_bytes;
      long long share = (region / gridDim.x + 15) & ~15LL;
      for (int s = 0; s < a.steps; ++s) {
        long long off = (long long)cta * share;
        long long len = off + share <= region ? share : region - off;
        const unsigned char* p = a.base + (long long)s * region + off;
        while (len > 0) { unsigned n = len > 16384 ? 16384u : (unsigned)len; prefetch_l2(p, n); p += n; len -= n; }
        // pace: stay `prefetch` steps ahead of the consumer (reads its progress through the empty barrier parity is not
        // visible here; a simple delay keeps the issue rate near the consumption rate)
        if (s >= a.prefetch) { const long long t0 = gt(); while (gt() - t0 < 300) {} }
      }
    } else {
      for (int strip = 0; strip < 6; ++strip) {  // each strip of 128 rows is one contiguous region
        const unsigned char* p = a.base + ((size_t)strip * gridDim.x + cta) * a.cta_bytes;
        for (long long off = 0; off < a.cta_bytes; off += 16384) prefetch_l2(p + off, 16384u);
        if (strip + 1 >= a.prefetch) { const long long t0 = gt(); while (gt() - t0 < 5000) {} }  // about one strip's time
      }
    }
  }
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int main(int argc, char** argv) {
  EncodeFn encode = nullptr;
  cudaDriverEntryPointQueryResult qres;
  CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", (void**)&encode, cudaEnableDefault, &qres));
  int sms = 0; CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
  const int NBUF = 3;
  const size_t bytes = 256ull << 20;
  unsigned char* bufs[NBUF];
  for (int i = 0; i < NBUF; ++i) { CK(cudaMalloc(&bufs[i], bytes)); CK(cudaMemset(bufs[i], i + 1, bytes)); }
  CK(cudaFuncSetAttribute(stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
  cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));

  struct Case { const char* name; int mode, ring, prefetch, promo; };
  const Case cases[] = {
      {"KN box [64k][96 cols] ring5", 0, 5, 0, 0}, {"KN box ring5 L2promo256", 0, 5, 0, 2}, {"KN box ring7", 0, 7, 0, 0},
      {"KN box ring5 + L2 prefetch 4 ahead", 0, 5, 4, 0}, {"KN box ring5 + L2 prefetch 8 ahead", 0, 5, 8, 0},
      {"packed [128 rows][128 B] ring5", 1, 5, 0, 0}, {"packed ring5 L2promo256", 1, 5, 0, 2}, {"packed ring10", 1, 10, 0, 0},
      {"packed ring5 + strip prefetch", 1, 5, 1, 0},
      {"packed 3-D box 4 chunks ring3", 2, 3, 0, 0}, {"packed 3-D box + strip prefetch", 2, 3, 1, 0},
      {"contiguous 1-D bulk 16 KB ring5", 3, 5, 0, 0}, {"contiguous 1-D bulk 16 KB ring10", 3, 10, 0, 0}, {"contiguous 1-D bulk 32 KB ring5", 4, 5, 0, 0},
  };
  for (const Case& c : cases) {
    Args a; memset(&a, 0, sizeof(a));
    a.mode = c.mode > 3 ? 3 : c.mode; a.ring = c.ring; a.prefetch = c.prefetch;
    CUtensorMap maps[NBUF]; memset(maps, 0, sizeof(maps));
    size_t total = 0;
    const CUtensorMapL2promotion promo = c.promo == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE;
    if (a.mode == 0) {
      const int K = 4096, N = sms * 96;
      a.cols = 96; a.steps = K / 64; a.stage_bytes = 64 * 96 * 4; a.row_bytes = (long long)N * 4;
      total = (size_t)K * N * 4;
      for (int i = 0; i < NBUF; ++i) {
        cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)K}; cuuint64_t strides[1] = {(cuuint64_t)N * 4};
        cuuint32_t box[2] = {96, 64}, el[2] = {1, 1};
        CUresult r = encode(&maps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, bufs[i], dims, strides, box, el, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { printf("encode failed %d\n", (int)r); return 1; }
      }
    } else if (a.mode == 1 || a.mode == 2) {
      const int rows = sms * 128 * 6, rowb = 2048;  // six strips of 128 rows per CTA
      a.cols = 128; a.row_bytes = rowb; a.cta_bytes = 128LL * rowb;
      total = (size_t)rows * rowb;
      for (int i = 0; i < NBUF; ++i) {
        CUresult r;
        if (a.mode == 1) {
          a.steps = 16 * 6; a.stage_bytes = 128 * 128;
          cuuint64_t dims[2] = {(cuuint64_t)rowb, (cuuint64_t)rows}; cuuint64_t strides[1] = {(cuuint64_t)rowb};
          cuuint32_t box[2] = {128, 128}, el[2] = {1, 1};
          r = encode(&maps[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, bufs[i], dims, strides, box, el, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        } else {
          a.steps = 4 * 6; a.stage_bytes = 128 * 128 * 4;
          cuuint64_t dims[3] = {128, (cuuint64_t)rows, 16}; cuuint64_t strides[2] = {(cuuint64_t)rowb, 128};
          cuuint32_t box[3] = {128, 128, 4}, el[3] = {1, 1, 1};
          r = encode(&maps[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, bufs[i], dims, strides, box, el, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        }
        if (r != CUDA_SUCCESS) { printf("encode failed %d\n", (int)r); return 1; }
      }
    } else {
      a.stage_bytes = c.mode == 4 ? 32768 : 16384; a.cta_bytes = 1536 * 1024; a.steps = (int)(a.cta_bytes / a.stage_bytes);
      total = (size_t)sms * a.cta_bytes;
    }
    const size_t smem = (size_t)a.ring * a.stage_bytes + 512;
    if (smem > 220 * 1024) { printf("%s: too much smem\n", c.name); continue; }
    float best = 1e9f, sum = 0; const int reps = 12;
    for (int it = 0; it < reps + 3; ++it) {
      a.base = bufs[it % NBUF];
      CK(cudaEventRecord(e0));
      stream_kernel<<<sms, 128, smem>>>(a, maps[it % NBUF]);
      CK(cudaEventRecord(e1));
      CK(cudaEventSynchronize(e1));
      float ms; CK(cudaEventElapsedTime(&ms, e0, e1));
      if (it >= 3) { sum += ms; if (ms < best) best = ms; }
    }
    CK(cudaGetLastError());
    unsigned fault = 0; CK(cudaMemcpyFromSymbol(&fault, g_fault, sizeof(fault)));
    printf("%-42s %7.1f MB  mean %7.2f us %7.1f GB/s   best %7.2f us %7.1f GB/s  fault %u\n", c.name, total / 1e6, sum / reps * 1e3,
           total / (sum / reps * 1e-3) * 1e-9, best * 1e3, total / (best * 1e-3) * 1e-9, fault);
    fflush(stdout);
  }
  return 0;
}
