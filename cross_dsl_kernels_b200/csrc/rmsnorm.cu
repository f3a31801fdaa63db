// Fused residual RMSNorm for sm_100a.
//
//   r = float(x) + float(residual);  y = T((r * rsqrt(mean(r^2) + eps)) * float(w));  r_out = T(r)
//
// One CTA owns one row and keeps the FP32 sum of the whole row in registers, so x and residual
// are read from HBM exactly once (128-bit streaming loads) and both outputs are written once
// (128-bit streaming stores): 4 * rows * hidden * sizeof(T) bytes of traffic, the algorithmic
// minimum.  The sum of squares is reduced with warp shuffles plus one shared-memory hop.
// The unrounded FP32 sum is what gets normalised; rounding to T happens only in the two stores.
#include <math.h>

#include "common.cuh"

namespace xdk {
namespace {

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* scratch /* THREADS/32 + 1 floats */) {
  v = warp_sum(v);
  if constexpr (THREADS == 32) return v;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < THREADS / 32 ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) scratch[THREADS / 32] = t;
  }
  __syncthreads();
  return scratch[THREADS / 32];
}

__device__ __forceinline__ float inv_rms(float sum_sq, float hidden_f, float eps) {
  // 1 / sqrt(mean + eps) with correctly rounded sqrt and divide, like the CPU reference's rsqrt.
  return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum_sq, hidden_f), eps)));
}

// Row-resident vector kernel: thread t holds vectors t, t+THREADS, ... (VPT of them) of the row.
template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
rmsnorm_row_kernel(const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ weight,
                   T* __restrict__ y, T* __restrict__ residual_out, int nvec, float hidden_f, float eps) {
  constexpr int E = Elem<T>::kPerVec;
  __shared__ float scratch[THREADS / 32 + 1];
  pdl_launch_dependents();
  const U4* wv = reinterpret_cast<const U4*>(weight);
  // Short rows (few vectors per thread) fetch the weight first: it is a constant operand, so the load may start
  // before the wait on the preceding kernel and is in flight during the reduction instead of after it.
  constexpr bool kEarlyWeight = VPT <= 4;
  U4 win[kEarlyWeight ? VPT : 1];
  if constexpr (kEarlyWeight) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * THREADS;
      if (v < nvec) win[i] = ld_cached16(wv + v);
    }
  }
  pdl_wait();  // x and residual may be the preceding kernel's output
  const size_t row_off = static_cast<size_t>(blockIdx.x) * nvec;  // in 16-byte vectors
  const U4* xv = reinterpret_cast<const U4*>(x) + row_off;
  const U4* rv = reinterpret_cast<const U4*>(residual) + row_off;
  U4* yv = reinterpret_cast<U4*>(y) + row_off;
  U4* ov = reinterpret_cast<U4*>(residual_out) + row_off;

  U4 xin[VPT], rin[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      xin[i] = ld_stream16(xv + v);
      rin[i] = ld_stream16(rv + v);
    }
  }
  float r[VPT][E];
  float sum_sq = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      float a[E], b[E];
      unpack16<T>(xin[i], a);
      unpack16<T>(rin[i], b);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        r[i][e] = __fadd_rn(a[e], b[e]);
        sum_sq = fmaf(r[i][e], r[i][e], sum_sq);
      }
      st_stream16(ov + v, pack16<T>(r[i]));
    }
  }
  const float scale = inv_rms(block_sum<THREADS>(sum_sq, scratch), hidden_f, eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      float w[E], out[E];
      if constexpr (kEarlyWeight) unpack16<T>(win[i], w);
      else unpack16<T>(ld_cached16(wv + v), w);
#pragma unroll
      for (int e = 0; e < E; ++e) out[e] = __fmul_rn(__fmul_rn(r[i][e], scale), w[e]);
      st_stream16(yv + v, pack16<T>(out));
    }
  }
}

// Any hidden, any alignment: two scalar passes; pass 2 re-reads x and residual (L2-resident by
// then) and recomputes the FP32 sum, it never reads back the rounded residual_out.
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_generic_kernel(const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ weight,
                       T* __restrict__ y, T* __restrict__ residual_out, int64_t hidden, float hidden_f,
                       float eps) {
  __shared__ float scratch[256 / 32 + 1];
  pdl_launch_dependents();
  pdl_wait();
  const size_t base = static_cast<size_t>(blockIdx.x) * hidden;
  float sum_sq = 0.0f;
  for (int64_t i = threadIdx.x; i < hidden; i += 256) {
    const float r = __fadd_rn(Elem<T>::to_f32(x[base + i]), Elem<T>::to_f32(residual[base + i]));
    residual_out[base + i] = Elem<T>::from_f32(r);
    sum_sq = fmaf(r, r, sum_sq);
  }
  const float scale = inv_rms(block_sum<256>(sum_sq, scratch), hidden_f, eps);
  for (int64_t i = threadIdx.x; i < hidden; i += 256) {
    const float r = __fadd_rn(Elem<T>::to_f32(x[base + i]), Elem<T>::to_f32(residual[base + i]));
    y[base + i] = Elem<T>::from_f32(__fmul_rn(__fmul_rn(r, scale), Elem<T>::to_f32(weight[i])));
  }
}

template <typename T, int THREADS, int VPT>
int launch_row(const void* x, const void* r, const void* w, void* y, void* ro, int64_t rows, int nvec,
               float hidden_f, float eps, cudaStream_t s) {
  return launch_dependent(rmsnorm_row_kernel<T, THREADS, VPT>, dim3(static_cast<unsigned>(rows)), dim3(THREADS), 0, s,
                static_cast<const T*>(x), static_cast<const T*>(r), static_cast<const T*>(w), static_cast<T*>(y),
                static_cast<T*>(ro), nvec, hidden_f, eps);
}

template <typename T>
int dispatch(const void* x, const void* r, const void* w, void* y, void* ro, int64_t rows, int64_t hidden, float eps,
             cudaStream_t s) {
  constexpr int E = Elem<T>::kPerVec;
  const float hidden_f = static_cast<float>(hidden);
  const bool vec_ok = hidden % E == 0 && aligned16(x) && aligned16(r) && aligned16(w) && aligned16(y) && aligned16(ro);
  const int64_t nvec = hidden / E;
  // Register budget: VPT * E floats of row state per thread; 16-bit types carry 8 per vector.
  const int64_t max_nvec = E == 4 ? 4096 : 2048;
  if (vec_ok && nvec <= max_nvec) {
    const int nv = static_cast<int>(nvec);
#define XDK_ROW(TH, V) return launch_row<T, TH, V>(x, r, w, y, ro, rows, nv, hidden_f, eps, s)
    if (nv <= 32) XDK_ROW(32, 1);
    if (nv <= 64) XDK_ROW(64, 1);
    if (nv <= 128) XDK_ROW(128, 1);
    if (nv <= 256) XDK_ROW(256, 1);
    if (nv <= 512) XDK_ROW(256, 2);
    if (nv <= 1024) XDK_ROW(256, 4);
    if (nv <= 2048) XDK_ROW(256, 8);
    if constexpr (E == 4) XDK_ROW(512, 8);
#undef XDK_ROW
  }
  return launch_dependent(rmsnorm_generic_kernel<T>, dim3(static_cast<unsigned>(rows)), dim3(256), 0, s,
                static_cast<const T*>(x), static_cast<const T*>(r), static_cast<const T*>(w), static_cast<T*>(y),
                static_cast<T*>(ro), hidden, hidden_f, eps);
}

}  // namespace
}  // namespace xdk

extern "C" int xdk_rmsnorm(const void* x, const void* residual, const void* weight, void* y, void* residual_out,
                           int64_t rows, int64_t hidden, float eps, int dtype, void* stream) {
  return xdk_rmsnorm_v2(x, residual, weight, y, residual_out, rows, hidden, eps, dtype, 0u, stream);
}

extern "C" int xdk_rmsnorm_v2(const void* x, const void* residual, const void* weight, void* y, void* residual_out,
                              int64_t rows, int64_t hidden, float eps, int dtype, unsigned flags, void* stream) {
  if (flags & ~XDK_DEPENDENT_LAUNCH) return XDK_ERR_ARG;
  xdk::CallFlagsScope scope(flags);
  if (!x || !residual || !weight || !y || !residual_out) return XDK_ERR_ARG;
  if (rows <= 0 || hidden <= 0 || !(eps > 0.0f) || !(eps < INFINITY)) return XDK_ERR_ARG;
  if (rows > 2147483647LL) return XDK_ERR_LIMIT;
  if (int st = xdk::require_sm100()) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case XDK_F32: return xdk::dispatch<float>(x, residual, weight, y, residual_out, rows, hidden, eps, s);
    case XDK_BF16: return xdk::dispatch<__nv_bfloat16>(x, residual, weight, y, residual_out, rows, hidden, eps, s);
    case XDK_F16: return xdk::dispatch<__half>(x, residual, weight, y, residual_out, rows, hidden, eps, s);
    default: return XDK_ERR_ARG;
  }
}
