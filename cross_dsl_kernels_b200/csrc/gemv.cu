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
  PeerOut out;  // y: the caller's buffer, or the same place in every rank's buffer
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
        peer_store(a.out, row0 + r, col0 + c, v);
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
      peer_store(a.out, row0 + r, col0 + c, v);
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
// M > 4: the op is bound by FP32 FMA issue (MT FMAs per weight element), so every SM has to get the
// same amount of work and its warps must never wait on global memory.
//
// Persistent kernel, one CTA per SM.  The weight matrix is cut into tiles of 32 k x 128 columns;
// tiles are numbered strip-major (all K tiles of column strip 0, then strip 1, ...) and CTA c takes
// the contiguous range [c*T/G, (c+1)*T/G): every CTA gets the same number of tiles (+-1) whatever
// N is.  A producer lane streams tiles with TMA tensor-map box copies (16 KB of W plus the matching
// 32-k slice of x, zero-filled outside M, N and K) into an 8-stage shared-memory ring; sixteen
// consumer warps each own one k-quad and one 64-column half of every tile and run pure shared-load +
// FMA code on an MT x 2 register tile (four warps per scheduler keep the FMA pipe busy).  KN tiles are read row-wise; NK tiles arrive 128-byte swizzled so that
// lanes reading different columns at the same k hit different banks.
// A strip that falls entirely inside one CTA's range is finished there (bias, store).  A strip cut
// by a range boundary leaves one partial [MT][128] per contributing CTA in the caller's scratch
// buffer and gemv_stream_finish_kernel adds them in CTA order: deterministic, no atomics.
constexpr int kTileK = 32, kTileN = 128;
constexpr int kTileStages = 8;
constexpr int kTileCtasPerSm = 1;
constexpr int kTileConsumers = 16;  // 8 k-quads x 2 column halves of a tile
constexpr int kTileThreads = (kTileConsumers + 1) * 32;
constexpr int kTileWBytes = kTileK * kTileN * 4;  // 16 KB

__device__ unsigned int g_gemv_fault;  // set when a bounded wait gives up

struct TileArgs {
  const float* bias;
  PeerOut out;
  float* scratch;  // [ctas][2][MT][128]
  int m, k, n;
  int strips, k_tiles;  // column strips, K tiles per strip
  int ctas;
};

__device__ __forceinline__ void tma_tile_2d(void* dst_smem, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst_smem)),
      "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kTileConsumers * 32) : "memory"); }

__host__ __device__ __forceinline__ int64_t tile_begin(int cta, int64_t total, int ctas) {
  return static_cast<int64_t>(cta) * total / ctas;
}

// Two independent FP32 FMAs in one instruction (sm_100): d.lo += a.lo*b.lo, d.hi += a.hi*b.hi, each
// rounded exactly like a scalar fma.rn.f32.
__device__ __forceinline__ void ffma2(float2& acc, float2 a, float2 b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;"
      : "+l"(reinterpret_cast<uint64_t&>(acc))
      : "l"(reinterpret_cast<const uint64_t&>(a)), "l"(reinterpret_cast<const uint64_t&>(b)));
}

template <int MT, bool NK>
__global__ void __launch_bounds__(kTileThreads, kTileCtasPerSm)
gemv_stream_kernel(TileArgs a, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap) {
  constexpr int kStageBytes = kTileWBytes + MT * kTileK * 4;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* ring = smem_raw;
  constexpr int RH = MT / 2;  // the cross-warp fold runs in two rounds of MT/2 rows to halve its buffer
  float* red = reinterpret_cast<float*>(smem_raw + kTileStages * kStageBytes);  // [8][MT/2][128]
  uint64_t* full = reinterpret_cast<uint64_t*>(red + 8 * RH * kTileN);
  uint64_t* empty = full + kTileStages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t total = static_cast<int64_t>(a.strips) * a.k_tiles;
  const int64_t t_begin = tile_begin(blockIdx.x, total, a.ctas), t_end = tile_begin(blockIdx.x + 1, total, a.ctas);

  if (threadIdx.x == 0) {
    for (int i = 0; i < kTileStages; ++i) {
      mbar_init(full + i, 1);
      mbar_init(empty + i, kTileConsumers);
    }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kTileConsumers) {
    // ---------------------------------------------------------------- producer (one lane)
    if (lane == 0) {
      int strip = static_cast<int>(t_begin / a.k_tiles);
      int kt = static_cast<int>(t_begin - static_cast<int64_t>(strip) * a.k_tiles);
      const int n_tiles = static_cast<int>(t_end - t_begin);
      for (int q = 0; q < n_tiles; ++q) {
        const int s = q % kTileStages;
        if (q >= kTileStages && !mbar_wait(empty + s, ((q / kTileStages) - 1) & 1)) {
          atomicOr(&g_gemv_fault, 1u);
          break;
        }
        unsigned char* dst = ring + s * kStageBytes;
        mbar_expect_tx(full + s, kStageBytes);
        if (NK) tma_tile_2d(dst, &wmap, kt * kTileK, strip * kTileN, full + s);
        else tma_tile_2d(dst, &wmap, strip * kTileN, kt * kTileK, full + s);
        tma_tile_2d(dst + kTileWBytes, &xmap, kt * kTileK, 0, full + s);
        if (++kt == a.k_tiles) kt = 0, ++strip;
      }
    }
  } else {
    // ---------------------------------------------------------------- consumers
    // KN: acc[r][c].x is the sum, .y unused.  NK: .x / .y are the partial sums over even / odd k, fed by
    // packed FMAs whose operand pairs (x[k],x[k+1]) and (w[k],w[k+1]) come straight out of 128-bit loads.
    const int kq = warp & 7, half_n = warp >> 3;  // this warp's k-quad and column half of every tile
    float2 acc[MT][2];
#pragma unroll
    for (int r = 0; r < MT; ++r)
#pragma unroll
      for (int c = 0; c < 2; ++c) acc[r][c] = make_float2(0.0f, 0.0f);
    bool ok = true;
    int strip = static_cast<int>(t_begin / a.k_tiles);
    int kt = static_cast<int>(t_begin - static_cast<int64_t>(strip) * a.k_tiles);
    const int first_strip = strip;
    const int n_tiles = static_cast<int>(t_end - t_begin);
    for (int q = 0; q < n_tiles; ++q) {
      const int s = q % kTileStages;
      if (ok && !mbar_wait(full + s, (q / kTileStages) & 1)) {
        ok = false;
        atomicOr(&g_gemv_fault, 2u);
      }
      if (ok) {
        const unsigned char* tile = ring + s * kStageBytes;
        const float* xs = reinterpret_cast<const float*>(tile + kTileWBytes);  // [MT][32]
        float wv[4][2];  // [k e][column c]
        if (NK) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int nloc = half_n * 64 + lane + 32 * c;
            const float4 v = *reinterpret_cast<const float4*>(tile + nloc * 128 + ((kq ^ (nloc & 7)) << 4));
            wv[0][c] = v.x, wv[1][c] = v.y, wv[2][c] = v.z, wv[3][c] = v.w;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 v = *reinterpret_cast<const float2*>(tile + (4 * kq + e) * (kTileN * 4) + half_n * 256 + lane * 8);
            wv[e][0] = v.x, wv[e][1] = v.y;
          }
        }
#pragma unroll
        for (int r = 0; r < MT; ++r) {
          const float4 t = *reinterpret_cast<const float4*>(xs + r * kTileK + 4 * kq);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            if (NK) {  // packed FMAs: .x / .y accumulate the even / odd k
              ffma2(acc[r][c], make_float2(t.x, t.y), make_float2(wv[0][c], wv[1][c]));
              ffma2(acc[r][c], make_float2(t.z, t.w), make_float2(wv[2][c], wv[3][c]));
            } else {
              acc[r][c].x = fmaf(t.x, wv[0][c], acc[r][c].x);
              acc[r][c].x = fmaf(t.y, wv[1][c], acc[r][c].x);
              acc[r][c].x = fmaf(t.z, wv[2][c], acc[r][c].x);
              acc[r][c].x = fmaf(t.w, wv[3][c], acc[r][c].x);
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
      }
      // ---- end of this CTA's share of the strip: fold the eight warps' sums and emit
      if (kt == a.k_tiles - 1 || q == n_tiles - 1) {
        const int64_t strip_first = static_cast<int64_t>(strip) * a.k_tiles;
        const bool whole = t_begin <= strip_first && t_end >= strip_first + a.k_tiles;
        const int slot = strip == first_strip ? 0 : 1;
        float* spill = a.scratch + (static_cast<size_t>(blockIdx.x) * 2 + slot) * MT * kTileN;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
          for (int r = 0; r < RH; ++r)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const int cl = half_n * 64 + (NK ? lane + 32 * c : lane * 2 + c);  // column inside the strip
              const float2 v = acc[half * RH + r][c];
              red[(kq * RH + r) * kTileN + cl] = NK ? v.x + v.y : v.x;
              acc[half * RH + r][c] = make_float2(0.0f, 0.0f);
            }
          consumer_sync();
          for (int o = threadIdx.x; o < RH * kTileN; o += kTileConsumers * 32) {
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; ++w) v += red[w * RH * kTileN + o];
            const int r = half * RH + o / kTileN, col = strip * kTileN + (o % kTileN);
            if (!whole) {
              spill[r * kTileN + (o % kTileN)] = v;
            } else if (r < a.m && col < a.n) {
              if (a.bias) v += a.bias[col];
              peer_store(a.out, r, col, v);
            }
          }
          consumer_sync();  // red is reused by the next round / strip
        }
      }
      if (++kt == a.k_tiles) kt = 0, ++strip;
    }
  }
}

// Adds, in CTA order, the partial sums of every strip that a range boundary cut.
template <int MT>
__global__ void __launch_bounds__(256)
gemv_stream_finish_kernel(TileArgs a) {
  const int strip = blockIdx.x;
  const int64_t total = static_cast<int64_t>(a.strips) * a.k_tiles;
  const int64_t first = static_cast<int64_t>(strip) * a.k_tiles, last = first + a.k_tiles;  // tile range of the strip
  // CTAs whose ranges overlap [first, last)
  int c_lo = static_cast<int>(first * a.ctas / total);
  while (c_lo > 0 && tile_begin(c_lo, total, a.ctas) > first) --c_lo;
  while (tile_begin(c_lo + 1, total, a.ctas) <= first) ++c_lo;
  int c_hi = c_lo;
  while (c_hi + 1 < a.ctas && tile_begin(c_hi + 1, total, a.ctas) < last) ++c_hi;
  if (c_lo == c_hi) return;  // the strip lay inside one CTA's range; that CTA wrote y itself
  // where each contributor parked its partial: slot 0 if this strip is the first of its range, else 1
  __shared__ const float* src[320];
  const int n_src = min(c_hi - c_lo + 1, 320);
  for (int i = threadIdx.x; i < n_src; i += 256) {
    const int c = c_lo + i;
    const int slot = strip == static_cast<int>(tile_begin(c, total, a.ctas) / a.k_tiles) ? 0 : 1;
    src[i] = a.scratch + (static_cast<size_t>(c) * 2 + slot) * MT * kTileN;
  }
  __syncthreads();
  for (int o = threadIdx.x; o < MT * kTileN; o += 256) {
    float v = 0.0f;
    for (int i = 0; i < n_src; ++i) v += src[i][o];
    const int r = o / kTileN, col = strip * kTileN + (o - r * kTileN);
    if (r < a.m && col < a.n) {
      if (a.bias) v += a.bias[col];
      peer_store(a.out, r, col, v);
    }
  }
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

template <int MT>
int launch_tile_stream(const float* x, const float* w, const float* bias, const PeerOut& out, int m, int k, int n, bool nk,
                       float* scratch, cudaStream_t stream) {
  TileArgs a;
  a.bias = bias, a.out = out, a.scratch = scratch;
  a.m = m, a.k = k, a.n = n;
  a.strips = (n + kTileN - 1) / kTileN;
  a.k_tiles = (k + kTileK - 1) / kTileK;
  const int64_t total = static_cast<int64_t>(a.strips) * a.k_tiles;
  const int64_t resident = static_cast<int64_t>(sm_count()) * kTileCtasPerSm;
  a.ctas = static_cast<int>(total < resident ? total : resident);
  CUtensorMap wmap, xmap;
  {
    const cuuint64_t dims_kn[2] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(k)};
    const cuuint64_t dims_nk[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(n)};
    const cuuint64_t stride_kn[1] = {static_cast<cuuint64_t>(n) * 4}, stride_nk[1] = {static_cast<cuuint64_t>(k) * 4};
    const cuuint32_t box_kn[2] = {kTileN, kTileK}, box_nk[2] = {kTileK, kTileN};
    const bool ok = nk ? encode_tiled_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, w, dims_nk, stride_nk, box_nk, true)
                       : encode_tiled_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, w, dims_kn, stride_kn, box_kn, false);
    const cuuint64_t xdims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(m)};
    const cuuint64_t xstride[1] = {static_cast<cuuint64_t>(k) * 4};
    const cuuint32_t xbox[2] = {kTileK, MT};
    if (!ok || !encode_tiled_2d(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, x, xdims, xstride, xbox, false)) return XDK_ERR_LAUNCH;
  }
  const size_t smem = static_cast<size_t>(kTileStages) * (kTileWBytes + MT * kTileK * 4) +
                      static_cast<size_t>(8) * (MT / 2) * kTileN * 4 + 2 * kTileStages * sizeof(uint64_t);
  int st;
  if (nk) {
    auto kernel = gemv_stream_kernel<MT, true>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) return note_launch(err);
    st = launch(kernel, dim3(a.ctas), dim3(kTileThreads), smem, stream, 1u, a, wmap, xmap);
  } else {
    auto kernel = gemv_stream_kernel<MT, false>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) return note_launch(err);
    st = launch(kernel, dim3(a.ctas), dim3(kTileThreads), smem, stream, 1u, a, wmap, xmap);
  }
  if (st != XDK_OK) return st;
  return launch(gemv_stream_finish_kernel<MT>, dim3(a.strips), dim3(256), 0, stream, 1u, a);
}

}  // namespace
}  // namespace xdk

namespace xdk {
namespace {

// ------------------------------------------------------------------------------------------------
// Scratch that lives in the library image instead of in caller-allocated memory.  Some hosts of
// this library cannot hand a kernel a workspace: a serving process that gave its whole device-memory
// budget to the KV cache at start-up and runs its decode loop with allocation switched off, or a
// plugin interface that passes inputs and outputs only.  For them xdk_gemv_f32_static_scratch runs the
// tile-stream kernel with its per-CTA partial sums parked in this array.  Every GPU that loads the
// library holds the 2.5 MB until the process exits.
constexpr int kStaticScratchCtas = 160;  // one CTA per SM; B200 has 148 SMs
constexpr size_t kStaticScratchFloats = static_cast<size_t>(kStaticScratchCtas) * 2 * 16 * kTileN;
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

// In host code the name above is only a stand-in for the symbol; the address a kernel can use has to
// be asked for, per device, with that device current.
float* static_scratch_for_current_device(int* status) {
  // Filled without locking: host threads that race here all store the same address.  Not refreshed after a
  // cudaDeviceReset() (the header says so).
  static float* address[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    *status = XDK_ERR_ARCH;
    return nullptr;
  }
  if (!address[dev]) {
    float* ptr = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
    if (err != cudaSuccess || !ptr) {
      *status = note_launch(err == cudaSuccess ? cudaErrorInvalidSymbol : err);
      return nullptr;
    }
    address[dev] = ptr;
  }
  *status = XDK_OK;
  return address[dev];
}

}  // namespace
}  // namespace xdk

extern "C" int xdk_gemv_f32_static_scratch(const float* x, const float* w, const float* bias, float* y, int64_t m,
                                           int64_t k, int64_t n, int weight_is_nk, void* stream) {
  using namespace xdk;
  if (!x || !w || !y) return XDK_ERR_ARG;
  if (m <= 4 || m > 16 || k <= 0 || n <= 0) return XDK_ERR_ARG;  // the tile-stream kernel covers 4 < M <= 16
  if (k >= (1 << 30) || n >= (1 << 30)) return XDK_ERR_LIMIT;
  const bool nk = weight_is_nk != 0;
  if (!aligned16(x) || !aligned16(w) || k % 4 != 0 || (!nk && n % 4 != 0)) return XDK_ERR_ARG;  // TMA-addressable operands
  if (int st = require_sm100()) return st;
  // the built-in array must hold two partial strips per CTA of this device
  if (xdk_gemv_scratch_bytes(m, k, n, weight_is_nk) > kStaticScratchFloats * sizeof(float)) return XDK_ERR_LIMIT;
  int st = XDK_OK;
  float* scratch = static_scratch_for_current_device(&st);
  if (!scratch) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const PeerOut out = single_out(y, n);
  return m > 8 ? launch_tile_stream<16>(x, w, bias, out, static_cast<int>(m), static_cast<int>(k), static_cast<int>(n), nk,
                                        scratch, s)
               : launch_tile_stream<8>(x, w, bias, out, static_cast<int>(m), static_cast<int>(k), static_cast<int>(n), nk,
                                       scratch, s);
}

namespace xdk {
unsigned gemv_fault_word() {
  unsigned v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemv_fault, sizeof(v)) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0x80000000u;
  }
  return v;
}
}  // namespace xdk

extern "C" int xdk_gemv_tc_plan(int64_t m, int64_t k, int64_t n, int weight_is_nk, int32_t* out5) {
  if (!out5) return XDK_ERR_ARG;
  return xdk::gemv_tc_plan(m, k, n, weight_is_nk != 0, out5);
}

extern "C" size_t xdk_gemv_scratch_bytes(int64_t m, int64_t k, int64_t n, int weight_is_nk) {
  (void)weight_is_nk;
  if (m <= 4 || m > 16 || k <= 0 || n <= 0) return 0;
  const int mt = m > 8 ? 16 : 8;
  return static_cast<size_t>(xdk::sm_count()) * xdk::kTileCtasPerSm * 2 * mt * xdk::kTileN * sizeof(float);
}

extern "C" int xdk_gemv_f32(const float* x, const float* w, const float* bias, float* y, int64_t m, int64_t k,
                            int64_t n, int weight_is_nk, int split_k, void* scratch, size_t scratch_bytes, void* stream) {
  // version 1 semantics: passing scratch asks for strict FP32 arithmetic
  return xdk_gemv_f32_v2(x, w, bias, y, m, k, n, weight_is_nk, split_k, scratch, scratch_bytes, scratch ? XDK_STRICT_FP32 : 0u,
                         stream);
}

extern "C" int xdk_gemv_f32_v2(const float* x, const float* w, const float* bias, float* y, int64_t m, int64_t k,
                               int64_t n, int weight_is_nk, int split_k, void* scratch, size_t scratch_bytes,
                               unsigned flags, void* stream) {
  if (!y || n <= 0) return XDK_ERR_ARG;
  xdk_peer_out one = {};
  one.ptr[0] = y, one.world = 1, one.ld = n, one.col0 = 0;
  return xdk_gemv_f32_peer(x, w, bias, &one, m, k, n, weight_is_nk, split_k, scratch, scratch_bytes, flags, stream);
}

extern "C" int xdk_gemv_f32_peer(const float* x, const float* w, const float* bias, const xdk_peer_out* y_out, int64_t m,
                                 int64_t k, int64_t n, int weight_is_nk, int split_k, void* scratch, size_t scratch_bytes,
                                 unsigned flags, void* stream) {
  using namespace xdk;
  if (flags & ~(XDK_STRICT_FP32 | XDK_DEPENDENT_LAUNCH)) return XDK_ERR_ARG;
  const bool strict = (flags & XDK_STRICT_FP32) != 0;
  PeerOut y;
  if (int st = make_out(y_out, nullptr, n, &y)) return st;
  if (!x || !w) return XDK_ERR_ARG;
  if (m <= 0 || k <= 0 || n <= 0) return XDK_ERR_ARG;
  if (!(split_k == 0 || split_k == 1 || split_k == 2 || split_k == 4 || split_k == 8)) return XDK_ERR_ARG;
  if (m > 16 * 65535LL || k > 2147483647LL - 4096 || n > 2147483647LL - 4096) return XDK_ERR_LIMIT;
  if (int st = require_sm100()) return st;
  const bool nk = weight_is_nk != 0;

  // 4 < M <= 16 unless strict FP32 was asked for: the tcgen05 kernel (split-TF32 products, FP32 accumulation; see
  // gemv_tc.cu).  Everything below this line is FP32 FMA arithmetic.
  if (split_k == 0 && !strict && gemv_tc_eligible(x, w, m, k, n, nk))
    return launch_gemv_tc(x, w, bias, y, static_cast<int>(m), static_cast<int>(k), static_cast<int>(n), nk,
                          static_cast<cudaStream_t>(stream));

  // 4 < M <= 16, a large weight matrix (the two extra launch/finish microseconds pay off from about
  // 48M elements), a scratch buffer and TMA-addressable operands: balanced persistent tile stream.
  if (split_k == 0 && m > 4 && m <= 16 && k * n >= (48LL << 20) && scratch && scratch_bytes >= xdk_gemv_scratch_bytes(m, k, n, weight_is_nk) &&
      aligned16(x) && aligned16(w) && aligned16(scratch) && k % 4 == 0 && (nk || n % 4 == 0) && k < (1 << 30) &&
      n < (1 << 30)) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return m > 8 ? launch_tile_stream<16>(x, w, bias, y, static_cast<int>(m), static_cast<int>(k), static_cast<int>(n), nk,
                                          static_cast<float*>(scratch), s)
                 : launch_tile_stream<8>(x, w, bias, y, static_cast<int>(m), static_cast<int>(k), static_cast<int>(n), nk,
                                         static_cast<float*>(scratch), s);
  }

  // Column strip width decides the grid: prefer the wide strip (128-bit loads in KN) whenever it
  // still yields enough CTAs to cover the machine; split-K multiplies the CTA count.
  const int mt = m >= 16 ? 16 : static_cast<int>(m);
  const int bn_wide = nk ? (mt > 4 ? 32 : 64) : 128;
  const int64_t strips_wide = (n + bn_wide - 1) / bn_wide;
  int splits = split_k;
  if (splits == 0) {
    // Smallest split that puts about 1.5 CTAs on every SM (2.7 for the KN kernels of M <= 4, whose 128-column strips
    // are few: K = 4096, N = 14336, M = 4 took 44.6 us with 224 CTAs and 40.9 with 448), as long as the whole grid is
    // resident at once: a second wave costs more than any split gains.
    const bool vec = aligned16(w) && aligned16(x) && k % 4 == 0 && (nk ? true : n % 4 == 0);
    const int ctas_per_sm = mt <= 2 ? 4 : (mt <= 4 ? (vec ? 4 : 3) : 2);  // register-limited residency of the MT variants
    const int64_t slots = static_cast<int64_t>(sm_count()) * ctas_per_sm;
    const int64_t want = (!nk && mt <= 4) ? 400 : 222;
    splits = 1;
    while (splits < 8 && strips_wide * splits < want && strips_wide * splits * 2 <= slots && k / (splits * 2) >= 256)
      splits *= 2;
  }
  const bool wide = nk || strips_wide * splits >= 96;
  const int64_t strips = wide ? strips_wide : (n + 31) / 32;
  if (strips > 2147483647LL) return XDK_ERR_LIMIT;

  GemvArgs a;
  a.x = x, a.w = w, a.bias = bias, a.out = y;
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
