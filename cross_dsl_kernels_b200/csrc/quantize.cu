// Device-side symmetric INT4 quantisation into the interchange format of the W4A16 projection.
//
// Bit-identical to the host function quantize_int4 (upstream src/crossdsl_kernels/quantization.py:39-63):
// per (row, group of `group` consecutive k)
//     peak  = max |w|                                   (FP32)
//     scale = half( peak == 0 ? 1 : max(peak / 7, 2^-24) )   -- rounded to FP16 BEFORE q is chosen
//     q     = clamp( rint(w / float(scale)), -7, 7 )    -- round half to even, like torch.round
//     code  = q + 8, two codes per byte, even k in the low nibble; an odd K pads the last high nibble with 8
// One warp owns one (row, group): every lane holds pairs (k, k + 1) so that it writes whole bytes.  The three
// conditions the host function raises on are reported through a status word instead (the caller reads it after
// the stream has drained): 1 = a weight is not finite, 2 = a scale is not representable in FP16, 4 = a
// dequantised weight half(q * scale) is not representable in FP16.
#include <math.h>

#include "common.cuh"

namespace xdk {
namespace {

template <typename T>
__global__ void __launch_bounds__(256)
quantize_int4_kernel(const T* __restrict__ w, uint8_t* __restrict__ packed, __half* __restrict__ scales,
                     int* __restrict__ status, int64_t n, int64_t k, int group, int64_t groups) {
  const int lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);  // (row, group)
  if (item >= n * groups) return;
  const int64_t row = item / groups, g = item - row * groups;
  const int64_t k0 = g * group;
  const T* src = w + row * k;
  const int64_t row_bytes = (k + 1) / 2;

  float v[8];  // pairs (k0 + 2 lane + 64 i, +1), i < group / 64 (group 32: lanes 0-15 only)
  float peak = 0.0f;
  int flags = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int off = 2 * lane + 64 * i + e;
      float x = 0.0f;
      if (off < group && k0 + off < k) x = Elem<T>::to_f32(src[k0 + off]);
      if (!isfinite(x)) flags |= 1;
      v[2 * i + e] = x;
      peak = fmaxf(peak, fabsf(x));
    }
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, s));
  const __half scale_h = peak == 0.0f ? __float2half_rn(1.0f) : __float2half_rn(fmaxf(__fdiv_rn(peak, 7.0f), 5.9604644775390625e-08f));
  const float scale = __half2float(scale_h);
  if (!isfinite(scale)) flags |= 2;
  if (lane == 0) scales[row * groups + g] = scale_h;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int off = 2 * lane + 64 * i;
    if (off < group && k0 + off < k) {
      int code[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float q = rintf(__fdiv_rn(v[2 * i + e], scale));
        q = fminf(fmaxf(q, -7.0f), 7.0f);
        if (!(q == q)) q = 0.0f;  // NaN from a non-finite weight or scale: already flagged
        if (!isfinite(__half2float(__float2half_rn(__fmul_rn(q, scale))))) flags |= 4;
        code[e] = static_cast<int>(q) + 8;
      }
      if (k0 + off + 1 >= k) code[1] = 8;  // pad nibble of an odd K
      packed[row * row_bytes + (k0 + off) / 2] = static_cast<uint8_t>(code[0] | (code[1] << 4));
    }
  }
  if (flags) atomicOr(status, flags);
}

}  // namespace
}  // namespace xdk

extern "C" int xdk_quantize_int4(const void* weight, int dtype, int64_t n, int64_t k, int group_size, uint8_t* packed,
                                 void* scales, int* status, void* stream) {
  using namespace xdk;
  if (!weight || !packed || !scales || !status) return XDK_ERR_ARG;
  if (n < 1 || k < 1) return XDK_ERR_ARG;
  if (!(group_size == 32 || group_size == 64 || group_size == 128 || group_size == 256)) return XDK_ERR_ARG;
  const int64_t groups = (k + group_size - 1) / group_size;
  if (n > (1LL << 40) / groups || (n * groups + 7) / 8 > 2147483647LL) return XDK_ERR_LIMIT;
  if (int st = require_sm100()) return st;
  const dim3 grid(static_cast<unsigned>((n * groups + 7) / 8));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  __half* sc = static_cast<__half*>(scales);
  switch (dtype) {
    case XDK_F32:
      return launch(quantize_int4_kernel<float>, grid, dim3(256), 0, s, 1u, static_cast<const float*>(weight), packed, sc,
                    status, n, k, group_size, groups);
    case XDK_BF16:
      return launch(quantize_int4_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, 1u,
                    static_cast<const __nv_bfloat16*>(weight), packed, sc, status, n, k, group_size, groups);
    case XDK_F16:
      return launch(quantize_int4_kernel<__half>, grid, dim3(256), 0, s, 1u, static_cast<const __half*>(weight), packed, sc,
                    status, n, k, group_size, groups);
    default:
      return XDK_ERR_ARG;
  }
}
