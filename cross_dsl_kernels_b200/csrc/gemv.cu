// FP32 decode projection  y[M,N] = x[M,K] W (+ bias)  for small M, sm_100a.
//
// The op is a weight stream: K*N*4 bytes of W are read once from HBM and everything else is
// noise, so the kernels are organised around keeping that stream coalesced and deep:
//   * KN ([K,N], N contiguous): lanes own adjacent columns (128-bit loads, 512 B per warp row),
//     the 8 warps of a CTA interleave over the K rows of the CTA's slice; partial sums meet in
//     shared memory at the end.
//   * NK ([N,K], K contiguous): a warp owns a few columns, lanes run along K (128-bit loads,
//     512 B per warp per column); partial sums meet through a shuffle reduce-scatter.
// Activations are staged per K-chunk into shared memory with cp.async (double-buffered), read
// back as 128-bit shared loads, and each weight element feeds MT strict-IEEE FP32 FMAs held in a
// register tile (MT rows x 4 columns per thread) -- no TF32, no tensor cores.
// Split-K: blockIdx.y indexes K slices; the slices of one column strip form a thread-block
// cluster and are summed in slice order through distributed shared memory, then bias is added
// once.  One launch, no scratch buffer, deterministic.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace xdk {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kChunk = 512;  // K elements of x staged per buffer

struct GemvArgs {
  const float* x;
  const float* w;
  const float* bias;
  float* y;
  int m, k, n;
  int k_slice;  // K elements per split-K slice (multiple of 32)
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Stage x[row0 .. row0+MT) x [k0, k0+kChunk) into xs[MT][kChunk]; rows >= m_valid and k >= k_end
// become zeros so the compute loop needs no predicates on x.
template <int MT, bool X16>
__device__ __forceinline__ void stage_x(float* xs, const float* x, int row0, int m_valid, int k, int k0, int k_end) {
  if constexpr (X16) {
    constexpr int kVecs = MT * kChunk / 4;
    for (int v = threadIdx.x; v < kVecs; v += kThreads) {
      const int r = v / (kChunk / 4), c = (v - r * (kChunk / 4)) * 4;
      float* dst = xs + r * kChunk + c;
      if (r < m_valid && k0 + c + 3 < k_end) {
        cp_async16(dst, x + static_cast<size_t>(row0 + r) * k + k0 + c);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          dst[e] = (r < m_valid && k0 + c + e < k_end) ? x[static_cast<size_t>(row0 + r) * k + k0 + c + e] : 0.0f;
      }
    }
  } else {
    for (int v = threadIdx.x; v < MT * kChunk; v += kThreads) {
      const int r = v / kChunk, c = v - r * kChunk;
      if (r < m_valid && k0 + c < k_end) {
        cp_async4(xs + v, x + static_cast<size_t>(row0 + r) * k + k0 + c);
      } else {
        xs[v] = 0.0f;
      }
    }
  }
  cp_async_commit();
}

// Sum NV per-lane values across the warp with a reduce-scatter (recursive halving): about NV
// shuffles instead of 5*NV.  On return element i of lane l is the warp total of original index
//   (l >> (5 - steps)) * (NV >> steps) + i,   steps = min(5, log2(NV)),
// and lanes that differ only in their low (5 - steps) bits hold identical copies.
template <int NV> __device__ __forceinline__ void warp_reduce_scatter(float (&v)[NV]) {
  static_assert((NV & (NV - 1)) == 0, "power of two");
  const int lane = threadIdx.x & 31;
  int cnt = NV;
#pragma unroll
  for (int mask = 16; mask > 0; mask >>= 1) {
    if (cnt > 1) {
      const int half = cnt / 2;
      const bool upper = (lane & mask) != 0;
#pragma unroll
      for (int i = 0; i < NV / 2; ++i) {
        if (i < half) {
          const float send = upper ? v[i] : v[i + half];
          const float keep = upper ? v[i + half] : v[i];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
        }
      }
      cnt = half;
    } else {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], mask);
    }
  }
}

// Final step shared by both layouts.  part[MT][BN] holds this CTA's partial sums for its strip and
// K slice.  With one slice the CTA writes y itself; with S slices the S CTAs of the cluster each
// finish a 1/S share of the strip, adding the S partials in slice order.
template <int MT, int BN>
__device__ __forceinline__ void finish_strip(float* part, const GemvArgs& a, int row0, int m_valid, int col0,
                                             int splits) {
  constexpr int kOut = MT * BN;
  if (splits == 1) {
    __syncthreads();
    for (int o = threadIdx.x; o < kOut; o += kThreads) {
      const int r = o / BN, c = o - r * BN;
      if (r < m_valid && col0 + c < a.n) {
        float v = part[o];
        if (a.bias) v += a.bias[col0 + c];
        a.y[static_cast<size_t>(row0 + r) * a.n + col0 + c] = v;
      }
    }
    return;
  }
  cg::cluster_group cluster = cg::this_cluster();
  cluster.sync();  // every slice's partial is in its CTA's shared memory
  const int rank = static_cast<int>(cluster.block_rank());
  const int share = kOut / splits;  // kOut is a multiple of 32, splits <= 8
  for (int i = threadIdx.x; i < share; i += kThreads) {
    const int o = rank * share + i;
    const int r = o / BN, c = o - r * BN;
    float v = 0.0f;
    for (int s = 0; s < splits; ++s) v += *cluster.map_shared_rank(part + o, s);
    if (r < m_valid && col0 + c < a.n) {
      if (a.bias) v += a.bias[col0 + c];
      a.y[static_cast<size_t>(row0 + r) * a.n + col0 + c] = v;
    }
  }
  cluster.sync();  // nobody leaves while a peer may still read its shared memory
}

// ------------------------------------------------------------------------------------------------
// KN layout.  CPT columns per lane (4: float4 loads; 1: scalar loads, for narrow grids).
// WVEC: W rows are 16-byte addressable (N % 4 == 0, aligned base) so CPT == 4 uses 128-bit loads.
template <int MT, int CPT, bool WVEC, bool X16>
__global__ void __launch_bounds__(kThreads)
gemv_kn_kernel(GemvArgs a) {
  constexpr int BN = 32 * CPT;
  extern __shared__ __align__(16) float smem[];
  float* xs = smem;                    // [2][MT][kChunk]
  float* part = smem + 2 * MT * kChunk;  // [MT][BN]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col0 = blockIdx.x * BN;
  const int col = col0 + lane * CPT;
  const int row0 = blockIdx.z * 16;
  const int m_valid = min(MT, a.m - row0);
  const int k_begin = blockIdx.y * a.k_slice;
  const int k_end = min(a.k, k_begin + a.k_slice);
  const int splits = gridDim.y;

  float acc[MT][CPT];
#pragma unroll
  for (int r = 0; r < MT; ++r)
#pragma unroll
    for (int c = 0; c < CPT; ++c) acc[r][c] = 0.0f;

  const int n_chunks = k_begin < k_end ? (k_end - k_begin + kChunk - 1) / kChunk : 0;
  if (n_chunks > 0) stage_x<MT, X16>(xs, a.x, row0, m_valid, a.k, k_begin, k_end);
  for (int ch = 0; ch < n_chunks; ++ch) {
    const int k0 = k_begin + ch * kChunk;
    float* xbuf = xs + (ch & 1) * MT * kChunk;
    if (ch + 1 < n_chunks) {
      stage_x<MT, X16>(xs + ((ch + 1) & 1) * MT * kChunk, a.x, row0, m_valid, a.k, k0 + kChunk, k_end);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // rows of this chunk in groups of 4; warp w takes groups w, w+8, ...; 2 groups per trip
    const int rows_here = min(kChunk, k_end - k0);
    const int groups = (rows_here + 3) / 4;
    constexpr int U = 2;
    for (int g = warp; g < groups; g += kWarps * U) {
      float wv[U][4][CPT];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int gk = (g + u * kWarps) * 4;  // row offset inside the chunk
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const bool row_ok = gk + j < rows_here;
          const float* wp = a.w + static_cast<size_t>(k0 + gk + j) * a.n + col;
          if constexpr (CPT == 4 && WVEC) {
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row_ok && col < a.n) t = ld_stream_f4(wp);
            wv[u][j][0] = t.x, wv[u][j][1] = t.y, wv[u][j][2] = t.z, wv[u][j][3] = t.w;
          } else {
#pragma unroll
            for (int c = 0; c < CPT; ++c) wv[u][j][c] = (row_ok && col + c < a.n) ? ld_stream_f1(wp + c) : 0.0f;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int gk = (g + u * kWarps) * 4;
        if (gk < rows_here) {
#pragma unroll
          for (int r = 0; r < MT; ++r) {
            const float4 xv = *reinterpret_cast<const float4*>(xbuf + r * kChunk + gk);
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
              acc[r][c] = fmaf(xv.x, wv[u][0][c], acc[r][c]);
              acc[r][c] = fmaf(xv.y, wv[u][1][c], acc[r][c]);
              acc[r][c] = fmaf(xv.z, wv[u][2][c], acc[r][c]);
              acc[r][c] = fmaf(xv.w, wv[u][3][c], acc[r][c]);
            }
          }
        }
      }
    }
    __syncthreads();  // chunk buffer free for the stage issued in the next trip
  }

  // cross-warp sum: red[warp][MT][BN] overlays the x buffers (8 * MT * BN <= 2 * MT * kChunk floats)
  float* red = smem;
#pragma unroll
  for (int r = 0; r < MT; ++r)
#pragma unroll
    for (int c = 0; c < CPT; ++c) red[(warp * MT + r) * BN + lane * CPT + c] = acc[r][c];
  __syncthreads();
  for (int o = threadIdx.x; o < MT * BN; o += kThreads) {
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) v += red[w * MT * BN + o];
    part[o] = v;
  }
  finish_strip<MT, BN>(part, a, row0, m_valid, col0, splits);
}

// ------------------------------------------------------------------------------------------------
// NK layout.  A warp owns CW columns; lanes run along K four elements at a time.
template <int MT, int CW, bool WVEC, bool X16>
__global__ void __launch_bounds__(kThreads)
gemv_nk_kernel(GemvArgs a) {
  constexpr int BN = kWarps * CW;
  extern __shared__ __align__(16) float smem[];
  float* xs = smem;
  float* part = smem + 2 * MT * kChunk;  // [MT][BN]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col0 = blockIdx.x * BN;
  const int colw = col0 + warp * CW;
  const int row0 = blockIdx.z * 16;
  const int m_valid = min(MT, a.m - row0);
  const int k_begin = blockIdx.y * a.k_slice;
  const int k_end = min(a.k, k_begin + a.k_slice);
  const int splits = gridDim.y;

  float acc[MT * CW];
#pragma unroll
  for (int i = 0; i < MT * CW; ++i) acc[i] = 0.0f;

  const int n_chunks = k_begin < k_end ? (k_end - k_begin + kChunk - 1) / kChunk : 0;
  if (n_chunks > 0) stage_x<MT, X16>(xs, a.x, row0, m_valid, a.k, k_begin, k_end);
  for (int ch = 0; ch < n_chunks; ++ch) {
    const int k0 = k_begin + ch * kChunk;
    float* xbuf = xs + (ch & 1) * MT * kChunk;
    if (ch + 1 < n_chunks) {
      stage_x<MT, X16>(xs + ((ch + 1) & 1) * MT * kChunk, a.x, row0, m_valid, a.k, k0 + kChunk, k_end);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int len = min(kChunk, k_end - k0);
    constexpr int U = 2;  // 2 steps of 128 k per trip
    for (int kk = 0; kk < len; kk += 128 * U) {
      float wv[U][CW][4];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int ko = kk + u * 128 + lane * 4;
#pragma unroll
        for (int c = 0; c < CW; ++c) {
          const float* wp = a.w + static_cast<size_t>(colw + c) * a.k + k0 + ko;
          const bool col_ok = colw + c < a.n;
          if constexpr (WVEC) {
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            if (col_ok && ko < len) t = ld_stream_f4(wp);  // len % 4 == 0 on this path
            wv[u][c][0] = t.x, wv[u][c][1] = t.y, wv[u][c][2] = t.z, wv[u][c][3] = t.w;
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) wv[u][c][e] = (col_ok && ko + e < len) ? ld_stream_f1(wp + e) : 0.0f;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int ko = kk + u * 128 + lane * 4;
        if (kk + u * 128 < len) {
#pragma unroll
          for (int r = 0; r < MT; ++r) {
            const float4 xv = *reinterpret_cast<const float4*>(xbuf + r * kChunk + ko);
#pragma unroll
            for (int c = 0; c < CW; ++c) {
              float s = acc[r * CW + c];
              s = fmaf(xv.x, wv[u][c][0], s);
              s = fmaf(xv.y, wv[u][c][1], s);
              s = fmaf(xv.z, wv[u][c][2], s);
              s = fmaf(xv.w, wv[u][c][3], s);
              acc[r * CW + c] = s;
            }
          }
        }
      }
    }
    __syncthreads();
  }

  warp_reduce_scatter<MT * CW>(acc);
  {
    constexpr int NV = MT * CW;
    constexpr int kSteps = NV >= 32 ? 5 : (NV == 16 ? 4 : (NV == 8 ? 3 : (NV == 4 ? 2 : (NV == 2 ? 1 : 0))));
    constexpr int kLeft = NV >> kSteps;  // values per writer lane
    if ((lane & ((1 << (5 - kSteps)) - 1)) == 0) {
#pragma unroll
      for (int i = 0; i < kLeft; ++i) {
        const int idx = (lane >> (5 - kSteps)) * kLeft + i;  // = r * CW + c
        const int r = idx / CW, c = idx - r * CW;
        part[r * BN + warp * CW + c] = acc[i];
      }
    }
  }
  __syncthreads();
  finish_strip<MT, BN>(part, a, row0, m_valid, col0, splits);
}

// ------------------------------------------------------------------------------------------------
// host side

template <int MT, int BNCOLS> constexpr size_t smem_bytes() { return (2 * MT * kChunk + MT * BNCOLS) * sizeof(float); }

template <typename Kernel>
int launch_gemv(Kernel kernel, size_t smem, const GemvArgs& a, int bn, int splits, cudaStream_t stream) {
  // Opt in to > 48 KB of dynamic shared memory (a per-function attribute; cheap to repeat).
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (err != cudaSuccess) return note_launch(err);
  dim3 grid((a.n + bn - 1) / bn, splits, (a.m + 15) / 16);
  return launch(kernel, grid, dim3(kThreads), smem, stream, static_cast<unsigned>(splits), a);
}

template <int MT>
int dispatch_mt(const GemvArgs& a, bool nk, int splits, bool wide, bool wvec, bool x16, cudaStream_t stream) {
#define XDK_GO(KERNEL, BN) return launch_gemv(KERNEL, smem_bytes<MT, BN>(), a, BN, splits, stream)
  if (!nk) {
    if (wide) {
      if (wvec && x16) XDK_GO((gemv_kn_kernel<MT, 4, true, true>), 128);
      if (wvec) XDK_GO((gemv_kn_kernel<MT, 4, true, false>), 128);
      if (x16) XDK_GO((gemv_kn_kernel<MT, 4, false, true>), 128);
      XDK_GO((gemv_kn_kernel<MT, 4, false, false>), 128);
    }
    if (x16) XDK_GO((gemv_kn_kernel<MT, 1, false, true>), 32);
    XDK_GO((gemv_kn_kernel<MT, 1, false, false>), 32);
  }
  constexpr int CW = MT >= 16 ? 4 : 8 / (MT >= 8 ? 2 : 1);  // keep MT*CW accumulators <= 64
  if (wvec && x16) XDK_GO((gemv_nk_kernel<MT, CW, true, true>), kWarps * CW);
  if (wvec) XDK_GO((gemv_nk_kernel<MT, CW, true, false>), kWarps * CW);
  if (x16) XDK_GO((gemv_nk_kernel<MT, CW, false, true>), kWarps * CW);
  XDK_GO((gemv_nk_kernel<MT, CW, false, false>), kWarps * CW);
#undef XDK_GO
}

}  // namespace
}  // namespace xdk

extern "C" int xdk_gemv_f32(const float* x, const float* w, const float* bias, float* y, int64_t m, int64_t k,
                            int64_t n, int weight_is_nk, int split_k, void* stream) {
  using namespace xdk;
  if (!x || !w || !y) return XDK_ERR_ARG;
  if (m <= 0 || k <= 0 || n <= 0) return XDK_ERR_ARG;
  if (!(split_k == 0 || split_k == 1 || split_k == 2 || split_k == 4 || split_k == 8)) return XDK_ERR_ARG;
  if (m > 16 * 65535LL || k > 2147483647LL - 4096 || n > 2147483647LL - 4096) return XDK_ERR_LIMIT;
  if (int st = require_sm100()) return st;
  const bool nk = weight_is_nk != 0;

  // Column strip width decides the grid: prefer the wide strip (128-bit loads in KN) whenever it
  // still yields enough CTAs to cover the machine; split-K multiplies the CTA count.
  const int mt = m >= 16 ? 16 : static_cast<int>(m);
  const int bn_wide = nk ? (mt > 4 ? 32 : 64) : 128;
  const int64_t strips_wide = (n + bn_wide - 1) / bn_wide;
  int splits = split_k;
  if (splits == 0) {
    splits = 1;
    while (splits < 8 && strips_wide * splits < 2 * 148 && k / (splits * 2) >= 256) splits *= 2;
  }
  const bool wide = nk || strips_wide * splits >= 96;
  const int64_t strips = wide ? strips_wide : (n + 31) / 32;
  if (strips > 2147483647LL) return XDK_ERR_LIMIT;

  GemvArgs a;
  a.x = x, a.w = w, a.bias = bias, a.y = y;
  a.m = static_cast<int>(m), a.k = static_cast<int>(k), a.n = static_cast<int>(n);
  const int64_t per = (k + splits - 1) / splits;
  a.k_slice = static_cast<int>((per + 31) / 32 * 32);
  const bool wvec = aligned16(w) && (nk ? k % 4 == 0 : n % 4 == 0);
  const bool x16 = aligned16(x) && k % 4 == 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (mt > 8) return dispatch_mt<16>(a, nk, splits, wide, wvec, x16, s);
  if (mt > 4) return dispatch_mt<8>(a, nk, splits, wide, wvec, x16, s);
  if (mt > 2) return dispatch_mt<4>(a, nk, splits, wide, wvec, x16, s);
  if (mt > 1) return dispatch_mt<2>(a, nk, splits, wide, wvec, x16, s);
  return dispatch_mt<1>(a, nk, splits, wide, wvec, x16, s);
}
