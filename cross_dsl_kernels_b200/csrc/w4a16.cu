// W4A16 projection  y[M,N] = half(x[M,K] W^T + bias),  W[n][k] = half((code - 8) * scale[n][k/g]).
//
// Weights arrive in the interchange format unchanged: uint8 [N, ceil(K/2)], low nibble = even k.
// A 16-byte load therefore carries 32 consecutive-k codes of one output column, and because every
// legal group size is a multiple of 32 those codes share one scale.  Codes are unpacked in
// registers with the FP16 "magic number" trick (or-ing a nibble into the mantissa of 1024.0 gives
// 1024 + code exactly), turned into code - 8 exactly, and multiplied by the FP16 scale with one
// FP16 rounding -- bit-identical to the format's definition half(float(q) * float(scale)), since
// that FP32 product is exact.  Products with x accumulate in FP32.
#include "common.cuh"

namespace xdk {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

struct W4Args {
  const __half* x;
  const uint8_t* packed;
  const __half* scales;
  const __half* bias;
  __half* y;
  int m, k, n;
  int group, groups;  // group size and scales per row
  int col_groups, groups_per_cta;
};

// Eight codes of one 32-bit word -> four half2 of dequantised weights, ordered
// (k0,k4) (k1,k5) (k2,k6) (k3,k7) relative to the word's first k.
__device__ __forceinline__ void dequant8(uint32_t word, __half2 scale2, __half2 (&w)[4]) {
  constexpr uint32_t kMagic = 0x64006400u;  // half2(1024, 1024)
  const uint32_t hi = word >> 8;
  uint32_t t0, t1, t2, t3;
  asm("lop3.b32 %0, %1, 0x000f000f, %2, 0xea;" : "=r"(t0) : "r"(word), "r"(kMagic));  // (a & b) | c
  asm("lop3.b32 %0, %1, 0x00f000f0, %2, 0xea;" : "=r"(t1) : "r"(word), "r"(kMagic));
  asm("lop3.b32 %0, %1, 0x000f000f, %2, 0xea;" : "=r"(t2) : "r"(hi), "r"(kMagic));
  asm("lop3.b32 %0, %1, 0x00f000f0, %2, 0xea;" : "=r"(t3) : "r"(hi), "r"(kMagic));
  const __half2 k1032 = __floats2half2_rn(1032.0f, 1032.0f);
  const __half2 k16th = __floats2half2_rn(0.0625f, 0.0625f);
  const __half2 km72 = __floats2half2_rn(-72.0f, -72.0f);
  // low nibbles: (1024 + c) - 1032 = c - 8;  high nibbles: (1024 + 16 c) / 16 - 72 = c - 8; both exact
  const __half2 q0 = __hsub2(*reinterpret_cast<__half2*>(&t0), k1032);
  const __half2 q1 = __hfma2(*reinterpret_cast<__half2*>(&t1), k16th, km72);
  const __half2 q2 = __hsub2(*reinterpret_cast<__half2*>(&t2), k1032);
  const __half2 q3 = __hfma2(*reinterpret_cast<__half2*>(&t3), k16th, km72);
  w[0] = __hmul2(q0, scale2);
  w[1] = __hmul2(q1, scale2);
  w[2] = __hmul2(q2, scale2);
  w[3] = __hmul2(q3, scale2);
}

// acc += a * b with FP16 operands and an FP32 accumulator in one instruction (sm_100 mixed FMA).
__device__ __forceinline__ void fma_h(float& acc, __half a, __half b) {
  asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(acc) : "h"(__half_as_ushort(a)), "h"(__half_as_ushort(b)));
}

// 16-byte units of x are XOR-swizzled in shared memory so that lanes reading consecutive
// 64-byte spans (32 halves each) hit distinct banks.
__device__ __forceinline__ int swz(int unit) { return unit ^ ((unit >> 3) & 3); }

// Fast SIMT path: K % 32 == 0, 16-byte aligned rows.  A warp owns CW columns at a time and lanes
// stride over the 16-byte vectors of the packed rows; x (all M rows, whole K) sits in shared memory.
template <int MT, int CW>
__global__ void __launch_bounds__(kThreads)
w4a16_simt_kernel(W4Args a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  U4* xs = reinterpret_cast<U4*>(smem_raw);  // [MT][K/8] swizzled 16-byte units
  const int units = a.k / 8;
  for (int i = threadIdx.x; i < MT * units; i += kThreads) {
    const int r = i / units, u = i - r * units;
    U4 v = U4{0u, 0u, 0u, 0u};
    if (r < a.m) v = ld_cached16(a.x + static_cast<size_t>(r) * a.k + u * 8);
    xs[r * units + swz(u)] = v;
  }
  __syncthreads();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int vecs = a.k / 32;         // 16-byte vectors per packed row
  const int row_bytes = a.k / 2;
  for (int gi = 0; gi < a.groups_per_cta; ++gi) {
    const int cg = blockIdx.x * a.groups_per_cta + gi;
    if (cg >= a.col_groups) break;
    const int col0 = (cg * kWarps + warp) * CW;
    float acc[MT][CW];
#pragma unroll
    for (int r = 0; r < MT; ++r)
#pragma unroll
      for (int c = 0; c < CW; ++c) acc[r][c] = 0.0f;

    for (int v0 = 0; v0 < vecs; v0 += 32 * 2) {
      U4 wv[2][CW];
      __half sc[2][CW];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int v = v0 + u * 32 + lane;
#pragma unroll
        for (int c = 0; c < CW; ++c) {
          const bool ok = v < vecs && col0 + c < a.n;
          wv[u][c] = U4{0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u};  // code 8 == weight 0
          sc[u][c] = __float2half(0.0f);
          if (ok) {
            wv[u][c] = ld_stream16(a.packed + static_cast<size_t>(col0 + c) * row_bytes + v * 16);
            sc[u][c] = __ldg(a.scales + static_cast<size_t>(col0 + c) * a.groups + (v * 32) / a.group);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int v = v0 + u * 32 + lane;
        if (v0 + u * 32 < vecs) {
          const int vv = v < vecs ? v : 0;  // out-of-range lanes multiply zeros by valid x
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // the four 32-bit words of the vector, 8 k each
            __half2 w[CW][4];
#pragma unroll
            for (int c = 0; c < CW; ++c) {
              const uint32_t word = j == 0 ? wv[u][c].x : (j == 1 ? wv[u][c].y : (j == 2 ? wv[u][c].z : wv[u][c].w));
              dequant8(word, __half2half2(sc[u][c]), w[c]);
            }
#pragma unroll
            for (int r = 0; r < MT; ++r) {
              const U4 xv = xs[r * units + swz(vv * 4 + j)];
              const __half* xh = reinterpret_cast<const __half*>(&xv);
#pragma unroll
              for (int c = 0; c < CW; ++c) {
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                  fma_h(acc[r][c], __low2half(w[c][p]), xh[p]);
                  fma_h(acc[r][c], __high2half(w[c][p]), xh[p + 4]);
                }
              }
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < MT; ++r)
#pragma unroll
      for (int c = 0; c < CW; ++c) {
        const float total = warp_sum(acc[r][c]);
        if (lane == 0 && r < a.m && col0 + c < a.n) {
          const float b = a.bias ? __half2float(a.bias[col0 + c]) : 0.0f;
          a.y[static_cast<size_t>(r) * a.n + col0 + c] = __float2half_rn(total + b);
        }
      }
  }
}

// Any K (odd included), any alignment: warp per column, lane per byte (two codes), rows one at a
// time.  Slow; it exists so that every shape the format allows has a GPU path.
__global__ void __launch_bounds__(kThreads)
w4a16_generic_kernel(W4Args a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * kWarps + warp;
  if (col >= a.n) return;
  const int row_bytes = (a.k + 1) / 2;
  for (int r = 0; r < a.m; ++r) {
    float acc = 0.0f;
    for (int b = lane; b < row_bytes; b += 32) {
      const uint32_t byte = a.packed[static_cast<size_t>(col) * row_bytes + b];
      const int k0 = 2 * b;
      const float s0 = __half2float(a.scales[static_cast<size_t>(col) * a.groups + k0 / a.group]);
      const float w0 = __half2float(__float2half_rn(__fmul_rn(static_cast<float>(static_cast<int>(byte & 15u) - 8), s0)));
      acc = fmaf(w0, __half2float(a.x[static_cast<size_t>(r) * a.k + k0]), acc);
      if (k0 + 1 < a.k) {
        const float s1 = __half2float(a.scales[static_cast<size_t>(col) * a.groups + (k0 + 1) / a.group]);
        const float w1 = __half2float(__float2half_rn(__fmul_rn(static_cast<float>(static_cast<int>(byte >> 4) - 8), s1)));
        acc = fmaf(w1, __half2float(a.x[static_cast<size_t>(r) * a.k + k0 + 1]), acc);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      const float b = a.bias ? __half2float(a.bias[col]) : 0.0f;
      a.y[static_cast<size_t>(r) * a.n + col] = __float2half_rn(acc + b);
    }
  }
}

template <int MT, int CW>
int launch_simt(W4Args a, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(MT) * a.k * sizeof(__half);
  auto kernel = w4a16_simt_kernel<MT, CW>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (err != cudaSuccess) return note_launch(err);
  a.col_groups = (a.n + kWarps * CW - 1) / (kWarps * CW);
  const int max_ctas = 2 * 148;
  a.groups_per_cta = (a.col_groups + max_ctas - 1) / max_ctas;
  const int ctas = (a.col_groups + a.groups_per_cta - 1) / a.groups_per_cta;
  return launch(kernel, dim3(ctas), dim3(kThreads), smem, stream, 1u, a);
}

}  // namespace
}  // namespace xdk

extern "C" int xdk_w4a16(const void* x, const uint8_t* packed, const void* scales, const void* bias, void* y,
                         int64_t m, int64_t k, int64_t n, int group_size, void* stream) {
  using namespace xdk;
  if (!x || !packed || !scales || !y) return XDK_ERR_ARG;
  if (m < 1 || m > 16 || k < 1 || n < 1) return XDK_ERR_ARG;
  if (!(group_size == 32 || group_size == 64 || group_size == 128 || group_size == 256)) return XDK_ERR_ARG;
  if (k >= (1LL << 31) || n >= (1LL << 31) || m * n >= (1LL << 31) || n * ((k + 1) / 2) >= (1LL << 31))
    return XDK_ERR_LIMIT;
  if (int st = require_sm100()) return st;
  W4Args a;
  a.x = static_cast<const __half*>(x);
  a.packed = packed;
  a.scales = static_cast<const __half*>(scales);
  a.bias = static_cast<const __half*>(bias);
  a.y = static_cast<__half*>(y);
  a.m = static_cast<int>(m), a.k = static_cast<int>(k), a.n = static_cast<int>(n);
  a.group = group_size;
  a.groups = static_cast<int>((k + group_size - 1) / group_size);
  a.col_groups = a.groups_per_cta = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool fast = k % 32 == 0 && aligned16(packed) && aligned16(x) && m * k * 2 <= 200 * 1024;
  if (fast) {
    if (m == 1) return launch_simt<1, 2>(a, s);
    if (m == 2) return launch_simt<2, 2>(a, s);
    if (m <= 4) return launch_simt<4, 2>(a, s);
    if (m <= 8) return launch_simt<8, 1>(a, s);
    return launch_simt<16, 1>(a, s);
  }
  return launch(w4a16_generic_kernel, dim3(static_cast<unsigned>((n + kWarps - 1) / kWarps)), dim3(kThreads), 0, s, 1u,
                a);
}
