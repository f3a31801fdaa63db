// W4A16 projection  y[M,N] = half(x[M,K] W^T + bias),  W[n][k] = half((code - 8) * scale[n][k/g]).
//
// Weights arrive in the interchange format unchanged: uint8 [N, ceil(K/2)], low nibble = even k.
// A 16-byte load therefore carries 32 consecutive-k codes of one output column, and because every
// legal group size is a multiple of 32 those codes share one scale.  Codes are unpacked in
// registers with the FP16 "magic number" trick (or-ing a nibble into the mantissa of 1024.0 gives
// 1024 + code exactly), turned into code - 8 exactly, and multiplied by the FP16 scale with one
// FP16 rounding -- bit-identical to the format's definition half(float(q) * float(scale)), since
// that FP32 product is exact.  Products with x accumulate in FP32.
//
// Compute paths (they share the unpack; the dispatcher at the end of the file picks one):
//   * M <= 8, K % 1024 == 0: mma.m16n8k16 with the operands swapped -- 16 weight columns are the MMA's rows, the rows of
//     x its columns -- fed from direct 16-byte loads (w4a16_mma_kernel).
//   * M >= 9 (and any M with a strided or multi-rank output), K % 256 == 0, group >= 64: tcgen05 kind::f16 with the
//     dequantised weights in tensor memory (w4a16_umma_kernel).
//   * shapes those two decline: a TMA-fed mma.sync stream kernel (M >= 3, K % 128 == 0), a SIMT kernel (lanes stride
//     over the packed row, mixed-precision FMAs, warp shuffle per column) and a generic kernel for any K.
// The k order inside an MMA fragment is free as long as both operands use the same order, so x is stored in shared
// memory pre-permuted to the order the unpack produces and no weight ever moves between lanes.
#include <cooperative_groups.h>
#include <stdlib.h>

#include "common.cuh"
#include "umma.cuh"

namespace cg = cooperative_groups;

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
  PeerOut out;        // where y goes for the tcgen05 kernel: y itself, or the same place in every rank's buffer
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
  extern __shared__ __align__(128) unsigned char smem_raw[];
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

// ------------------------------------------------------------------------------------------------
// Tensor-core building blocks.  A warp works on blocks of 8 columns in steps of 128 k: in a step
// lane (g = lane/4, j = lane%4) holds the 16 bytes with k in [32j, 32j+32) of column g of the block.
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Physical position of 16-byte unit `unit` of x row `row`: the XOR spreads the eight units a
// quarter-warp reads in one shared-memory phase (2 rows x 4 lanes) over all eight bank groups.
__device__ __forceinline__ int xunit(int unit, int row) { return unit ^ ((((unit >> 3) & 1) << 1) | (row & 1)); }

// ------------------------------------------------------------------------------------------------
// Streaming tensor-core path (the one used for 3 <= M <= 16 when K % 128 == 0).
//
// One persistent CTA per SM.  The N/8 column blocks are dealt out evenly to clusters of S CTAs
// (S = split-K factor, 1/2/4); inside a cluster CTA r takes the K chunks r, r+S, ... of 1024 k, and
// inside a CTA warp w takes blocks w, w+8, ...  A (chunk, block) tile is 8 column rows of 512 packed
// bytes plus their scales.  Every warp runs its own software pipeline: an elected lane keeps the TMA
// box copies (one op for the weights, one for the scales) of the warp's next three tiles in flight
// into a private four-slot shared-memory ring, completing on per-slot mbarriers, while the warp
// unpacks the current tile in registers and feeds mma.m16n8k16.  (A warp can only keep a handful
// of ordinary load instructions in flight; one TMA op moves a whole 4 KB tile.)  x for the current chunk sits in shared memory, pre-permuted and swizzled
// as in the path above and double-buffered across chunks.  Partial sums of the S CTAs meet through
// distributed shared memory in rank order.
constexpr int kStreamWarps = 8;
constexpr int kStreamThreads = kStreamWarps * 32;
constexpr int kChunkK = 1024;                       // k per chunk
constexpr int kRowStride = kChunkK / 2;             // a tile is a dense TMA box: 8 column rows x 512 B
constexpr int kSlotBytes = 8 * kRowStride + 512;    // + up to 8 x 64 B of scales (dense box, 8 rows)
// ring slots per warp: all but one hold tiles in flight; 16 staged x rows leave room for 3, 8 rows for 4
// MR = rows of x staged per chunk (8 for M <= 8, else 16)
template <int MR> struct StreamDepth { static constexpr int value = MR == 16 ? 3 : 4; };
constexpr int kMaxNB = 8;                           // column blocks per warp per pass

__device__ unsigned int g_w4_fault;  // set when a bounded wait gives up

struct StreamPlan {
  int clusters;        // number of clusters (grid = clusters * splits)
  int splits;          // CTAs per cluster = split-K factor
  int total_blocks;    // ceil(N / 8)
  int chunks;          // ceil(K / 1024)
  int ring_scales;     // 1: the chunk's scales travel through the ring with the weights
};

template <int MR>
__global__ void __launch_bounds__(kStreamThreads, 1)
w4a16_stream_kernel(W4Args a, StreamPlan plan, const __grid_constant__ CUtensorMap wmap,
                    const __grid_constant__ CUtensorMap smap) {
  constexpr bool ROWS16 = MR == 16;
  constexpr int kRows = MR;
  constexpr int kXUnits = kChunkK / 8;  // 16-byte units per staged x row
  constexpr int kPassBlocks = kStreamWarps * kMaxNB;
  constexpr int kDepth = StreamDepth<MR>::value;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, j = lane & 3;
  unsigned char* ring = smem_raw + warp * kDepth * kSlotBytes;                          // this warp's slots
  U4* xs = reinterpret_cast<U4*>(smem_raw + kStreamWarps * kDepth * kSlotBytes);       // [2][kRows][kXUnits]
  float* part = reinterpret_cast<float*>(smem_raw + kStreamWarps * kDepth * kSlotBytes + 2 * kRows * kChunkK * 2);
  uint64_t* full = reinterpret_cast<uint64_t*>(part + 16 * kStreamWarps * kMaxNB * 8) + warp * kDepth;  // this warp's barriers
  if (lane == 0) {
    for (int i = 0; i < kDepth; ++i) mbar_init(full + i, 1);
    mbar_fence_init();
  }
  __syncwarp();

  const int rank = plan.splits > 1 ? static_cast<int>(cg::this_cluster().block_rank()) : 0;
  const int cluster_id = blockIdx.x / plan.splits;
  // even deal of column blocks to clusters
  const int blk_begin = static_cast<int>(static_cast<int64_t>(cluster_id) * plan.total_blocks / plan.clusters);
  const int blk_end = static_cast<int>(static_cast<int64_t>(cluster_id + 1) * plan.total_blocks / plan.clusters);
  const int nblk = blk_end - blk_begin;
  const int my_chunks = plan.chunks > rank ? (plan.chunks - rank + plan.splits - 1) / plan.splits : 0;
  const int row_bytes = a.k / 2;
  const int scale_shift = 31 - __clz(a.group);  // group is a power of two

  // ---- prefetch side: walks the same (pass, chunk, block) sequence as the compute loop, ahead of it
  int pf_p0 = 0, pf_ci = 0, pf_b = warp, pf_q = 0;
  bool pf_valid = my_chunks > 0 && nblk > 0;
  auto pf_normalize = [&]() {
    while (pf_valid && pf_b >= min(kPassBlocks, nblk - pf_p0)) {
      pf_b = warp;
      if (++pf_ci >= my_chunks) {
        pf_ci = 0;
        pf_p0 += kPassBlocks;
        if (pf_p0 >= nblk) pf_valid = false;
      }
    }
  };
  const unsigned tile_bytes = 8 * kRowStride + (plan.ring_scales ? 8u * ((kChunkK >> scale_shift) * 2) : 0u);
  auto pf_issue = [&]() {  // TMA ops for the next tile of this warp (if any) into slot pf_q % kDepth
    pf_normalize();
    if (pf_valid) {
      if (lane == 0) {
        const int kc = rank + pf_ci * plan.splits;
        const int col0 = (blk_begin + pf_p0 + pf_b) * 8;
        unsigned char* dst = ring + (pf_q % kDepth) * kSlotBytes;
        uint64_t* bar = full + pf_q % kDepth;
        mbar_expect_tx(bar, tile_bytes);  // out-of-range parts of a box are zero-filled and still counted
        tma_box_2d(dst, &wmap, kc * (kChunkK / 8), col0, bar);
        if (plan.ring_scales) tma_box_2d(dst + 8 * kRowStride, &smap, kc * (kChunkK >> scale_shift), col0, bar);
      }
      pf_b += kStreamWarps;
      ++pf_q;
    }
  };
#pragma unroll
  for (int d = 0; d < kDepth - 1; ++d) pf_issue();

  int q = 0;  // tiles this warp has consumed
  for (int p0 = 0; p0 < nblk; p0 += kPassBlocks) {
    const int nb_pass = min(kPassBlocks, nblk - p0);
    const int cols = nb_pass * 8;  // width of part[16][cols] for this pass

    // x staging.  A thread owns kStage 16-byte units of every chunk.  The first chunk of a pass is
    // staged at once; the next chunk is staged two units at a time around the tiles of the current
    // one (loads issued before a tile, permuted and stored after it) so that only two units are
    // ever live in registers during the unpack/mma loop.
    constexpr int kStage = (kRows * kXUnits + kStreamThreads - 1) / kStreamThreads;  // units per thread per chunk
    auto x_load = [&](int kc, int i) -> U4 {
      const int idx = threadIdx.x + i * kStreamThreads;
      const int r = idx / kXUnits, u = idx - r * kXUnits;
      const int k0 = kc * kChunkK + u * 8;
      U4 v = U4{0u, 0u, 0u, 0u};
      if (idx < kRows * kXUnits && r < a.m && k0 < a.k) v = ld_cached16(a.x + static_cast<size_t>(r) * a.k + k0);
      return v;
    };
    auto x_store = [&](int buf, int i, const U4& t) {
      const int idx = threadIdx.x + i * kStreamThreads;
      if (idx >= kRows * kXUnits) return;
      const int r = idx / kXUnits, u = idx - r * kXUnits;
      U4 v;  // the unpack's k order (0,4,1,5,2,6,3,7) inside every 8-block
      v.x = __byte_perm(t.x, t.z, 0x5410);
      v.y = __byte_perm(t.x, t.z, 0x7632);
      v.z = __byte_perm(t.y, t.w, 0x5410);
      v.w = __byte_perm(t.y, t.w, 0x7632);
      xs[(buf * kRows + r) * kXUnits + xunit(u, r)] = v;
    };
    if (my_chunks > 0) {
      U4 first[kStage];
#pragma unroll
      for (int i = 0; i < kStage; ++i) first[i] = x_load(rank, i);
#pragma unroll
      for (int i = 0; i < kStage; ++i) x_store(0, i, first[i]);
    }
    __syncthreads();

    for (int ci = 0; ci < my_chunks; ++ci) {
      const int kc = rank + ci * plan.splits;
      const int steps = min(kChunkK, a.k - kc * kChunkK) / 128;
      const bool more = ci + 1 < my_chunks;
      const bool last = !more;
      int staged = more ? 0 : kStage;  // units of the next chunk this thread has staged so far
      const U4* xb = xs + (ci & 1) * kRows * kXUnits;
      for (int b = warp; b < nb_pass; b += kStreamWarps, ++q) {
        const bool stage_now = staged < kStage;
        U4 nx0 = U4{0u, 0u, 0u, 0u}, nx1 = U4{0u, 0u, 0u, 0u};
        if (stage_now) {
          nx0 = x_load(kc + plan.splits, staged);
          nx1 = x_load(kc + plan.splits, staged + 1);
        }
        {
          const int col = (blk_begin + p0 + b) * 8 + g;
          // Slow path only (scales not in the ring): this lane's scale for every step, fetched before the wait
          __half sc[8];
          if (!plan.ring_scales) {
  #pragma unroll
            for (int st = 0; st < 8; ++st) {
              sc[st] = __float2half(0.0f);
              if (st < steps && col < a.n)
                sc[st] = __ldg(a.scales + static_cast<size_t>(col) * a.groups + ((kc * kChunkK + st * 128 + j * 32) >> scale_shift));
            }
          }
          pf_issue();  // refill the slot freed by the previous tile
          const bool landed = mbar_wait(full + q % kDepth, (q / kDepth) & 1);
          const unsigned char* slot = ring + (q % kDepth) * kSlotBytes;
          const unsigned char* tile = slot + g * kRowStride + j * 16;
          const __half* tile_scales =
              reinterpret_cast<const __half*>(slot + 8 * kRowStride + g * ((kChunkK >> scale_shift) * 2));
          if (!landed) atomicOr(&g_w4_fault, 1u);
          float part4[8][4];  // eight independent accumulator chains hide the mma latency
  #pragma unroll
          for (int w = 0; w < 8; ++w)
  #pragma unroll
            for (int e = 0; e < 4; ++e) part4[w][e] = 0.0f;
  #pragma unroll
          for (int st = 0; st < 8; ++st) {
            if (st >= steps || !landed) break;
            U4 wv = U4{0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u};
            __half s1 = __float2half(0.0f);
            if (col < a.n) {
              wv = *reinterpret_cast<const U4*>(tile + st * 64);
              s1 = plan.ring_scales ? tile_scales[(st * 128 + j * 32) >> scale_shift] : sc[st];
            }
            const __half2 s2 = __half2half2(s1);
  #pragma unroll
            for (int w = 0; w < 4; ++w) {
              const int unit = st * 16 + j * 4 + w;
              const U4 xa = xb[g * kXUnits + xunit(unit, g)];
              U4 xc = U4{0u, 0u, 0u, 0u};
              if constexpr (ROWS16) xc = xb[(g + 8) * kXUnits + xunit(unit, g + 8)];
              const uint32_t word = w == 0 ? wv.x : (w == 1 ? wv.y : (w == 2 ? wv.z : wv.w));
              __half2 h[4];
              dequant8(word, s2, h);
              mma16816(part4[2 * w], xa.x, xc.x, xa.y, xc.y, *reinterpret_cast<uint32_t*>(&h[0]),
                       *reinterpret_cast<uint32_t*>(&h[1]));
              mma16816(part4[2 * w + 1], xa.z, xc.z, xa.w, xc.w, *reinterpret_cast<uint32_t*>(&h[2]),
                       *reinterpret_cast<uint32_t*>(&h[3]));
            }
          }
          __syncwarp();  // every lane is done reading the slot before the next pf_issue overwrites it

          // C[row g][2j], C[g][2j+1], C[g+8][2j], C[g+8][2j+1] of this block for this chunk
          float c4[4];
  #pragma unroll
          for (int e = 0; e < 4; ++e)
            c4[e] = ((part4[0][e] + part4[1][e]) + (part4[2][e] + part4[3][e])) + ((part4[4][e] + part4[5][e]) + (part4[6][e] + part4[7][e]));
          float* mine = part + g * cols + b * 8 + 2 * j;  // rows g and g+8 of part[16][cols]; only this lane touches them
          if (ci > 0) {
            c4[0] += mine[0], c4[1] += mine[1];
            c4[2] += mine[8 * cols], c4[3] += mine[8 * cols + 1];
          }
          if (last && plan.splits == 1) {
  #pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int row = g + (e >> 1) * 8, oc = (blk_begin + p0 + b) * 8 + 2 * j + (e & 1);
              if (row < a.m && oc < a.n) {
                const float bv = a.bias ? __half2float(a.bias[oc]) : 0.0f;
                a.y[static_cast<size_t>(row) * a.n + oc] = __float2half_rn(c4[e] + bv);
              }
            }
          } else {
            mine[0] = c4[0], mine[1] = c4[1];
            mine[8 * cols] = c4[2], mine[8 * cols + 1] = c4[3];
          }
        }
        if (stage_now) {
          x_store((ci + 1) & 1, staged, nx0);
          x_store((ci + 1) & 1, staged + 1, nx1);
          staged += 2;
        }
      }
      for (; staged < kStage; ++staged) x_store((ci + 1) & 1, staged, x_load(kc + plan.splits, staged));
      __syncthreads();
    }
  }
  if (plan.splits > 1) {
    // The host guarantees a single pass when K is split, so part[16][nblk * 8] is complete here.
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int cols = nblk * 8;
    const int total = 16 * cols;
    const int share = (total + plan.splits - 1) / plan.splits;
    for (int i = threadIdx.x; i < share; i += kStreamThreads) {
      const int o = rank * share + i;
      if (o < total) {
        const int row = o / cols, c = o - row * cols;
        const int col = blk_begin * 8 + c;
        float v = 0.0f;
        for (int sidx = 0; sidx < plan.splits; ++sidx) v += *cluster.map_shared_rank(part + o, sidx);
        if (row < a.m && col < a.n) {
          const float bv = a.bias ? __half2float(a.bias[col]) : 0.0f;
          a.y[static_cast<size_t>(row) * a.n + col] = __float2half_rn(v + bv);
        }
      }
    }
    cluster.sync();
  }
}

template <int MR>
int launch_stream(const W4Args& a, cudaStream_t stream) {
  const int sms = xdk::sm_count();
  StreamPlan plan;
  plan.total_blocks = (a.n + 7) / 8;
  plan.chunks = (a.k + kChunkK - 1) / kChunkK;
  plan.ring_scales = (a.group <= 128 && a.k % kChunkK == 0 && aligned16(a.scales)) ? 1 : 0;
  constexpr int kDepth = StreamDepth<MR>::value;
  const size_t smem = static_cast<size_t>(kStreamWarps) * kDepth * kSlotBytes + 2 * MR * kChunkK * 2 +
                      16 * kStreamWarps * kMaxNB * 8 * sizeof(float) + kStreamWarps * kDepth * sizeof(uint64_t);
  CUtensorMap wmap, smap;
  {
    // packed weights as a [N][K/8] matrix of 32-bit words; box = 8 rows x 128 words (1024 k)
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.k / 8), static_cast<cuuint64_t>(a.n)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.k / 2)};
    const cuuint32_t box[2] = {kChunkK / 8, 8};
    if (!encode_tiled(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, a.packed, dims, strides, box, false)) return XDK_ERR_LAUNCH;
    smap = wmap;
    if (plan.ring_scales) {
      const cuuint64_t sdims[2] = {static_cast<cuuint64_t>(a.groups), static_cast<cuuint64_t>(a.n)};
      const cuuint64_t sstrides[1] = {static_cast<cuuint64_t>(a.groups) * 2};
      const cuuint32_t sbox[2] = {static_cast<cuuint32_t>(kChunkK / a.group), 8};
      if (!encode_tiled(&smap, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, a.scales, sdims, sstrides, sbox, false)) return XDK_ERR_LAUNCH;
    }
  }
  auto kernel = w4a16_stream_kernel<MR>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (err != cudaSuccess) return note_launch(err);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kStreamThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;

  // How many clusters of S CTAs fit on the device at once (1 CTA per SM; a cluster must sit inside
  // one GPC, so this is not simply SMs / S).  Asked once per S, then cached.
  static int resident[3] = {0, 0, 0};  // S = 1, 2, 4
  auto resident_clusters = [&](int s_log2) {
    if (resident[s_log2] == 0) {
      const int sz = 1 << s_log2;
      int n = 0;
      if (sz == 1) {
        n = sms;
      } else {
        cfg.gridDim = dim3(sms / sz * sz);
        attr[0].val.clusterDim.x = sz;
        cfg.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
          (void)cudaGetLastError();
          n = 0;
        }
      }
      resident[s_log2] = n > 0 ? n : -1;
    }
    return resident[s_log2] > 0 ? resident[s_log2] : 0;
  };
  // Split K over a cluster so that each CTA stages only 1/S of x, as long as (a) the whole grid stays
  // resident in one wave, (b) it does not idle more than ~6 % of the SMs, and (c) the cluster can
  // finish its blocks in one pass (partial sums are parked in shared memory).
  int best_log2 = 0;
  for (int s_log2 = 2; s_log2 >= 1; --s_log2) {
    const int sz = 1 << s_log2;
    if (sz > plan.chunks) continue;
    const int fit = resident_clusters(s_log2);
    if (fit * sz * 100 < sms * 94) continue;
    const int clusters = min(fit, plan.total_blocks);
    if ((plan.total_blocks + clusters - 1) / clusters > kStreamWarps * kMaxNB) continue;
    best_log2 = s_log2;
    break;
  }
  plan.splits = 1 << best_log2;
  plan.clusters = min(resident_clusters(best_log2), plan.total_blocks);
  if (plan.clusters <= 0) plan.clusters = min(sms, plan.total_blocks), plan.splits = 1;
  cfg.gridDim = dim3(plan.clusters * plan.splits);
  attr[0].val.clusterDim.x = plan.splits;
  cfg.numAttrs = plan.splits > 1 ? 1 : 0;
  return note_launch(cudaLaunchKernelEx(&cfg, kernel, a, plan, wmap, smap));
}


// ------------------------------------------------------------------------------------------------
// tcgen05 path (M > 8, K % 256 == 0, group >= 64): the contraction runs on the 5th-generation tensor
// cores.  Operands are swapped so that the UMMA "M" dimension (128 TMEM lanes) carries output columns:
//     D[128 lanes x 16 S] += A[128 x 16 k] * B[16 k x 16 S],   A = dequantised W,  B = x^T
// and A lives in TENSOR MEMORY: the unpack warps write the dequantised weights straight from registers
// into TMEM (tcgen05.st), so they never pass through shared memory.  (With A in shared memory every
// M=128,N=16 MMA re-reads 4 KB of A for 16 columns of use, which by itself saturates the 128 B/clk
// shared-memory port and starves the unpack warps that share it.)
//
// One persistent CTA per SM owns a contiguous, evenly dealt range of 32-column units and walks it in
// strips of <= 4 units, full K each (no cross-CTA reduction).  A warp may touch only the TMEM lane quarter
// warp % 4, so a strip narrower than 128 columns would leave unpack warps idle.  Instead K is split S ways
// over the lane quarters (S = 4 for a 1-unit strip, 2 for 2 units, 1 otherwise): quarter lq holds columns
// of unit lq % (4/S) for the k range lq / (4/S), and B gets 16 S rows, rows 16 ks .. 16 ks + 15 being x over
// k range ks.  An MMA then multiplies every lane with every k range; lane quarter lq keeps only the block of
// 16 accumulator columns that belongs to its own range, and the S partial sums of a column meet in shared
// memory in a fixed order.  (N = 64 costs the tensor pipe no more than N = 16 here: the MMA rate is bound by
// issue, see below.)
//   TMA warp, one lane : box copies of the packed codes of a (strip, 256-k step): one 4 KB, 128-byte swizzled
//                        box per live lane quarter, into a ring of step buffers; plus the strip's scales
//   x warps (2)        : one lane issues one TMA box per k range ([16 rows][256 k], 512-byte rows; a box whose
//                        inner extent is one 16-byte unit would land the operand layout directly, but TMA moves
//                        such boxes unit by unit and was slower than the whole unpack); both warps then move every
//                        16-byte unit to its place in the canonical K-major core-matrix layout ([k group][8 rows]
//                        [8 k]), reordering its 8 k to the order the unpack produces, and hand the buffer to the MMAs
//   unpack warps (8)   : thread = one TMEM lane; warp w owns lane quarter w % 4 and k half w / 4 of every step:
//                        16-byte shared loads of codes -> dequant -> tcgen05.st
//   MMA warps (4)      : one lane each.  A warp gets a tcgen05.mma out only every ~100 cycles, whatever the shape
//                        (measured: 94-118 cycles per M=128 MMA for N = 16 .. 128), while four warps issuing side
//                        by side reach one per ~29 cycles.  So the 16 K=16 blocks of a step are dealt round-robin
//                        to 4 issuers, each accumulating into its OWN accumulator, then tcgen05.commit onto the
//                        barriers (count 4) that hand the stage / x buffer back and announce the finished strip
//   unpack warps 0-3   : epilogue -- tcgen05.ld of the four accumulators, summed in fixed order, (S > 1: the
//                        k-range partials through shared memory,) bias, FP16 store
// TMEM columns (512 allocated; the kernel is alone on its SM): 64 i .. accumulator of issuer i (16 S used),
// 256 + 128 s .. A stage s.
// Every wait is time-bounded; on a timeout the kernel raises g_w4_fault, stops issuing work, and still
// frees its TMEM columns before it returns.
constexpr int kUStepK = 256;                   // k per step: one packed box row (128 bytes), one A stage
constexpr int kUPackedBufs = 4;                // packed steps in flight (16 KB each)
constexpr int kUMaxStages = 3;                 // A operand stages in TMEM: 3 while the accumulators fit 128 columns, else 2
constexpr int kUMaxXBufs = 4;                  // x step buffers (raw and operand layout each): 4 unless a strip splits K four ways
constexpr int kUIssuers = 4;                   // MMA-issuing warps, one accumulator each
constexpr int kUTmemCols = 512;                // allocation (power of two): accumulators first, then the stages
constexpr int kUStageCols = kUStepK / 2;       // 32-bit TMEM columns per stage (two FP16 k per column)
constexpr int kUXLbo = 128, kUXSbo = (kUStepK / 8) * kUXLbo;  // x: [row group of 8][32 k groups][8 rows x 16 B]
constexpr int kUXBytes = 8 * kUXSbo;           // an x buffer for 64 rows (S = 4); the x region is 2 x 2 of these
constexpr int kUXRegion = 2 * kUXBytes;        // bytes of all operand images (and again of all raw buffers)
constexpr int kUPackedBytes = 4 * 32 * (kUStepK / 2);  // 4 lane quarters x 32 rows x 128 B
constexpr int kURedBytes = 128 * 16 * 4;       // k-range partials: [lane][16] floats
constexpr int kWTma = 8, kWMma0 = 9, kWX0 = 10, kWMma1 = 12;  // warp roles; 0-7 unpack, 10-11 x, 12-14 MMA
constexpr int kUThreads = 15 * 32;

struct UmmaPlan {
  int ctas, total_units;  // 32-column units
  int smax;               // widest K split (lane quarters) any strip of the launch uses: sizes the x buffers
  int xdepth;             // x buffers in flight: the x region cut into buffers of smax x 8 KB, at most kUMaxXBufs
  int stages;             // A stages in TMEM
};

__global__ void __launch_bounds__(kUThreads, 1)
w4a16_umma_kernel(W4Args a, UmmaPlan plan, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap,
                  const __grid_constant__ CUtensorMap xmap) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* packed = smem_raw;                                 // [kUPackedBufs][kUPackedBytes]
  // A step's x is smax k ranges of [16 rows][256 k] = smax x 8 KB, raw as TMA lands it and again as operand image.
  // With a small smax the same memory holds more steps: the x path (TMA -> x warps -> MMA -> buffer free) is a loop of
  // ~1.4 us, which with two buffers set the step time of the whole kernel.
  const int xstride = plan.smax * 2 * kUXSbo, xdepth = plan.xdepth;
  const int kUStages = plan.stages;
  const int kUAccCols = (kUTmemCols - kUStages * kUStageCols) / kUIssuers, kUTmemA = kUIssuers * kUAccCols;
  unsigned char* xbuf = packed + kUPackedBufs * kUPackedBytes;      // [xdepth][xstride] operand images
  unsigned char* xraw = xbuf + kUXRegion;                           // [xdepth][smax k ranges][16 rows][256 k] as TMA lands it
  unsigned char* scbuf = xraw + kUXRegion;                          // [128 lanes][scale_row_bytes]
  const int scale_row_bytes = a.groups * 2;
  float* red = reinterpret_cast<float*>(scbuf + 128 * scale_row_bytes);  // [128 lanes][16]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(red) + kURedBytes);
  uint64_t* pk_full = bars;                       // [kUPackedBufs]  TMA bytes of a packed step landed
  uint64_t* pk_empty = pk_full + kUPackedBufs;    // [kUPackedBufs]  the 8 unpack warps are done with the step
  uint64_t* a_full = pk_empty + kUPackedBufs;     // [kUMaxStages] the 8 unpack warps wrote the stage to TMEM
  uint64_t* a_empty = a_full + kUMaxStages;       // [kUMaxStages] every issuer's MMAs that read the stage completed
  uint64_t* x_raw = a_empty + kUMaxStages;        // [kUMaxXBufs] TMA bytes of an x step landed
  uint64_t* x_full = x_raw + kUMaxXBufs;          // [kUMaxXBufs] both x warps reordered their share
  uint64_t* x_empty = x_full + kUMaxXBufs;        // [kUMaxXBufs] every issuer's MMAs that read the buffer completed
  uint64_t* sc_full = x_empty + kUMaxXBufs;       // [1]
  uint64_t* acc_full = sc_full + 1;               // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int scale_shift = 31 - __clz(a.group);
  UmmaCursor cur;
  cur.init(blockIdx.x, plan.ctas, plan.total_units, a.k, kUStepK);

  if (threadIdx.x == 0) {
    pdl_launch_dependents();  // the next kernel of the stream may be scheduled (it waits for this one's data itself)
    for (int i = 0; i < kUPackedBufs; ++i) {
      mbar_init(pk_full + i, 1);
      mbar_init(pk_empty + i, 8);   // one arrival per unpack warp
    }
    for (int i = 0; i < xdepth; ++i) {
      mbar_init(x_raw + i, 1);
      mbar_init(x_full + i, 1);     // one x thread, after the x warps met
      mbar_init(x_empty + i, kUIssuers);
    }
    for (int i = 0; i < kUStages; ++i) {
      mbar_init(a_full + i, 8);
      mbar_init(a_empty + i, kUIssuers);
    }
    mbar_init(sc_full, 1);
    mbar_init(acc_full, kUIssuers);
    mbar_fence_init();
  }
  if (warp == kWMma0) {  // TMEM: accumulators + A stages
    tmem_alloc<kUTmemCols>(tmem_slot);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kWTma) {
    // ------------------------------------------------------------ TMA producer: packed codes and scales
    {  // the whole warp runs the loop (waits included), one elected lane issues: operands stay warp-uniform
      bool ok = true;
      int strip_i = 0;
      while (ok && cur.begin_strip()) {
        const int qpk = 4 / cur.split;  // lane quarters per k range = units the strip can hold
        // scales of the strip (whole K, once per live lane quarter): the buffer is free once the unpack warps
        // have released the last packed step of the previous strip
        if (strip_i > 0) {
          const int prev = cur.q - 1;
          ok = __all_sync(0xffffffffu, mbar_wait(pk_empty + prev % kUPackedBufs, (prev / kUPackedBufs) & 1));
          if (!ok) break;
        }
        if (elect_one()) {
          mbar_expect_tx(sc_full, static_cast<unsigned>(cur.units * cur.split * 32 * scale_row_bytes));
          for (int lq = 0; lq < 4; ++lq)
            if (lq % qpk < cur.units) tma_box_2d(scbuf + lq * 32 * scale_row_bytes, &smap, 0, (cur.unit + lq % qpk) * 32, sc_full);
        }
        __syncwarp();
        do {
          const int buf = cur.q % kUPackedBufs;
          if (cur.q >= kUPackedBufs) {
            ok = __all_sync(0xffffffffu, mbar_wait(pk_empty + buf, ((cur.q / kUPackedBufs) - 1) & 1));
            if (!ok) break;
          }
          if (elect_one()) {
            mbar_expect_tx(pk_full + buf, static_cast<unsigned>(cur.units * cur.split * 32 * (kUStepK / 2)));
            for (int lq = 0; lq < 4; ++lq)  // 32-row boxes; the 128-byte swizzle depends on (row & 7) only
              if (lq % qpk < cur.units)
                tma_box_2d(packed + buf * kUPackedBytes + lq * 32 * (kUStepK / 2), &wmap,
                           ((lq / qpk) * cur.kper + cur.kc * kUStepK) / 8, (cur.unit + lq % qpk) * 32, pk_full + buf);
          }
          __syncwarp();
        } while (cur.next_step());
        ++strip_i;
      }
      if (!ok && lane == 0) atomicOr(&g_w4_fault, 4u);
    }
  } else if (warp == kWMma0 || warp >= kWMma1) {
    // ------------------------------------------------------------ MMA issuers
    {  // whole warp, one elected lane issues (a lane-0-only loop issued a tcgen05.mma only every ~120 ns)
      const int issuer = warp == kWMma0 ? 0 : warp - kWMma1 + 1;
      const uint32_t acc = tmem_base + issuer * kUAccCols;
      // x descriptor: only the 14-bit start-address field changes from MMA to MMA
      const uint64_t xd0 = umma_desc(smem_u32(xbuf), kUXLbo, kUXSbo);
      const uint32_t xd_lo = static_cast<uint32_t>(xd0), xd_hi = static_cast<uint32_t>(xd0 >> 32);
      bool ok = true;
      RingPos xp, sp;
      while (ok && cur.begin_strip()) {
        // D = F32, A = B = F16 K-major, N = 16 S, M = 128
        const uint32_t idesc = umma_idesc(16 * cur.split, 0u);
        do {
          const int xb = xp.slot, s = sp.slot;
          ok = __all_sync(0xffffffffu, mbar_wait(x_full + xb, xp.parity) && mbar_wait(a_full + s, sp.parity));
          if (!ok) break;
          xp.advance(xdepth), sp.advance(kUStages);
          tc_fence_after();
          const uint32_t a_base = tmem_base + kUTmemA + s * kUStageCols + issuer * 8;
          const uint32_t x_lo = xd_lo + ((xb * xstride + issuer * 2 * kUXLbo) >> 4);
          if (elect_one()) {
#pragma unroll
            for (int j = 0; j < kUStepK / 16 / kUIssuers; ++j) {  // K blocks issuer, issuer + 4, ...
              uint64_t xd;
              asm("mov.b64 %0, {%1, %2};" : "=l"(xd) : "r"(x_lo + ((j * kUIssuers * 2 * kUXLbo) >> 4)), "r"(xd_hi));
              umma_f16_ta(acc, a_base + j * kUIssuers * 8, xd, idesc, !(cur.kc == 0 && j == 0));
            }
            umma_commit(a_empty + s);   // the TMEM stage is free once every issuer's MMAs have read it
            umma_commit(x_empty + xb);
          }
          __syncwarp();
        } while (cur.next_step());
        if (ok && elect_one()) umma_commit(acc_full);
        __syncwarp();
      }
      if (!ok && lane == 0) atomicOr(&g_w4_fault, 8u);
    }
  } else if (warp >= kWX0) {
    // ------------------------------------------------------------ x warps
    const int t = threadIdx.x - kWX0 * 32;  // 0 .. 63
    bool ok = true;
    UmmaCursor ahead = cur;  // issues the loads, xdepth steps in front of `cur`
    bool ahead_live = ahead.begin_strip();
    RingPos xi, xs;          // of the load being issued, of the step being reordered
    auto issue = [&]() {  // raw buffer xi.slot is free: its last readers passed the x-warp barrier
      if (!ahead_live) return;
      if (t == 0) {
        const int xb = xi.slot;
        mbar_expect_tx(x_raw + xb, static_cast<unsigned>(ahead.split * 16 * kUStepK * 2));
        for (int ks = 0; ks < ahead.split; ++ks)  // rows >= M are out of range: zero-filled, still counted
          tma_box_2d(xraw + xb * xstride + ks * 16 * kUStepK * 2, &xmap, ks * ahead.kper + ahead.kc * kUStepK, 0, x_raw + xb);
      }
      xi.advance(xdepth);
      if (!ahead.next_step()) ahead_live = ahead.begin_strip();
    };
    if (t == 0) pdl_wait();  // x is the preceding kernel's output; packed codes and scales (issued already) are not
    for (int i = 0; i < xdepth; ++i) issue();
    // A quarter warp moves an 8-row x 8-k-group block per pass along its diagonals: lane i takes k group i of row
    // (i + r) & 7, so the eight 16-byte loads (row pitch 512 B) and the eight stores (k-group pitch 128 B) each hit
    // eight different bank groups.
    const int qw = t >> 3, li = t & 7;        // 8 quarter warps: (row group, quarter of the 32 k groups)
    const int mg = qw >> 2, kg = (qw & 3) * 8 + li;
    while (cur.begin_strip()) {
      do {
        const int xb = xs.slot;
        if (ok) ok = mbar_wait(x_raw + xb, xs.parity);
        if (ok) ok = mbar_wait(x_empty + xb, xs.parity ^ 1u);  // a fresh barrier passes: nothing has read the buffer yet
        xs.advance(xdepth);
        if (ok) {
          auto fetch = [&](int ks, U4 (&v)[8]) {
            const unsigned char* src = xraw + xb * xstride + ks * 16 * kUStepK * 2 + kg * 16;
#pragma unroll
            for (int r = 0; r < 8; ++r) v[r] = *reinterpret_cast<const U4*>(src + (mg * 8 + ((li + r) & 7)) * (kUStepK * 2));
          };
          auto place = [&](int ks, const U4 (&v)[8]) {
            unsigned char* dst = xbuf + xb * xstride + (ks * 2 + mg) * kUXSbo + kg * kUXLbo;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
              U4 o;  // k 0..7 of one row -> 0,4,1,5,2,6,3,7, the order the unpack produces
              o.x = __byte_perm(v[r].x, v[r].z, 0x5410);
              o.y = __byte_perm(v[r].x, v[r].z, 0x7632);
              o.z = __byte_perm(v[r].y, v[r].w, 0x5410);
              o.w = __byte_perm(v[r].y, v[r].w, 0x7632);
              *reinterpret_cast<U4*>(dst + ((li + r) & 7) * 16) = o;
            }
          };
          if (cur.split == 1) {
            U4 v[8];
            fetch(0, v);
            place(0, v);
          } else {
            // a step of a strip that splits K carries 2 or 4 k ranges of x: two at a time, so that the two x warps
            // have sixteen loads in flight instead of eight (the x path sets the step time of these strips)
            for (int ks = 0; ks < cur.split; ks += 2) {
              U4 va[8], vb[8];
              fetch(ks, va);
              fetch(ks + 1, vb);
              place(ks, va);
              place(ks + 1, vb);
            }
          }
          fence_async_smem();
        }
        asm volatile("bar.sync 2, 64;" ::: "memory");  // both x warps are done with the raw buffer and wrote their share
        if (t == 0) mbar_arrive_cta(x_full + xb);
        issue();
      } while (cur.next_step());
    }
    if (!ok && lane == 0) atomicOr(&g_w4_fault, 32u);
  } else {
    // ------------------------------------------------------------ unpack warps (+ epilogue)
    const int lq = warp & 3, kh = warp >> 2;  // TMEM lane quarter this warp may touch, k half of a step
    const int c = lq * 32 + lane;             // this thread's TMEM lane
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(lq * 32) << 16);
    const uint32_t a_lane_base = lane_base + kUTmemA + kh * (kUStageCols / 2);
    const __half* sc_row = reinterpret_cast<const __half*>(scbuf + c * scale_row_bytes);
    int strip_i = 0;
    bool ok = true;
    RingPos sp;
    while (cur.begin_strip()) {
      const int qpk = 4 / cur.split;
      const int ks = lq / qpk, uq = lq % qpk;   // this quarter's k range and unit of the strip
      const bool warp_live = uq < cur.units;    // warp-uniform: a quarter without columns writes nothing
      const int col = (cur.unit + uq) * 32 + lane;  // output column of this thread
      const int k_range0 = ks * cur.kper;
      const int split = cur.split;
      if (ok) ok = mbar_wait(sc_full, strip_i & 1);
      do {
        const int buf = cur.q % kUPackedBufs, s = sp.slot;
        if (ok) ok = mbar_wait(pk_full + buf, (cur.q / kUPackedBufs) & 1);
        if (ok) ok = mbar_wait(a_empty + s, sp.parity ^ 1u);
        sp.advance(kUStages);
        if (ok && warp_live) {
          tc_fence_after();
          // packed tiles arrive 128-byte swizzled: 16-byte piece p of row r sits at piece p ^ (r & 7), so the
          // lanes of a warp, which read the same piece of 32 different rows, spread over all bank groups
          const unsigned char* row = packed + buf * kUPackedBytes + c * (kUStepK / 2);
          const int k_half = k_range0 + cur.kc * kUStepK + kh * (kUStepK / 2);
#pragma unroll
          for (int pp = 0; pp < kUStepK / 128; ++pp) {  // two pieces = 64 k = 32 TMEM columns per store
            // (a tcgen05.st costs the warp ~125 ns whatever its width, so 32 columns go out at once)
            uint32_t r[32];
            // two pieces = 64 k lie inside one group (group >= 64)
            const __half2 s2 = __half2half2(sc_row[(k_half + pp * 64) >> scale_shift]);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const int piece = kh * (kUStepK / 64) + pp * 2 + half;
              const U4 wv = *reinterpret_cast<const U4*>(row + ((piece ^ (c & 7)) << 4));  // rows past N are zero-filled: harmless
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                const uint32_t word = w == 0 ? wv.x : (w == 1 ? wv.y : (w == 2 ? wv.z : wv.w));
                __half2 h[4];
                dequant8(word, s2, h);
#pragma unroll
                for (int i = 0; i < 4; ++i) r[16 * half + 4 * w + i] = *reinterpret_cast<uint32_t*>(&h[i]);
              }
            }
            tmem_st32(a_lane_base + s * kUStageCols + pp * 32, r);
          }
          tmem_wait_st();
          tc_fence_before();
        }
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_cta(a_full + s);
          mbar_arrive_cta(pk_empty + buf);
        }
      } while (cur.next_step());
      // ---- epilogue of the strip: warps 0-3 read their own lane quarter of the four accumulators
      float sum[16];
      if (warp < 4) {
        if (ok) ok = mbar_wait(acc_full, strip_i & 1);
        if (ok && warp_live) {
          tc_fence_after();
#pragma unroll
          for (int i = 0; i < kUIssuers; ++i) {
            uint32_t r[16];
            tmem_ld16(lane_base + i * kUAccCols + ks * 16, r);  // the 16 accumulator columns of this quarter's own k range
#pragma unroll
            for (int m = 0; m < 16; ++m) sum[m] = i == 0 ? __uint_as_float(r[m]) : __fadd_rn(sum[m], __uint_as_float(r[m]));
          }
          tc_fence_before();
          if (split > 1) {
#pragma unroll
            for (int m = 0; m < 16; m += 4)
              *reinterpret_cast<float4*>(red + c * 16 + m) = make_float4(sum[m], sum[m + 1], sum[m + 2], sum[m + 3]);
          }
        }
      }
      if (split > 1) {
        asm volatile("bar.sync 1, 256;" ::: "memory");  // strip-uniform: the k-range partials are in shared memory
        if (warp < 4 && ok && warp_live && ks == 0) {
          for (int j = 1; j < split; ++j)  // fixed order: k range 0 + 1 + 2 + 3
#pragma unroll
            for (int m = 0; m < 16; ++m) sum[m] = __fadd_rn(sum[m], red[(c + j * qpk * 32) * 16 + m]);
        }
      }
      if (warp < 4 && ok && warp_live && ks == 0 && col < a.n) {
        const float bv = a.bias ? __half2float(a.bias[col]) : 0.0f;
#pragma unroll
        for (int m = 0; m < 16; ++m)
          if (m < a.m) peer_store(a.out, m, col, __float2half_rn(sum[m] + bv));
      }
      // all 256 threads meet before the next strip's stages can reach the MMA warps (a_full needs all of them),
      // so the next strip's first MMAs cannot overwrite TMEM (nor its partials the shared buffer) while they are read
      asm volatile("bar.sync 1, 256;" ::: "memory");
      ++strip_i;
    }
    if (!ok && lane == 0) atomicOr(&g_w4_fault, 16u);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kWMma0) {
    tc_fence_after();
    tmem_dealloc<kUTmemCols>(tmem_base);
  }
}

int launch_umma(const W4Args& a, bool dependent, cudaStream_t stream) {
  UmmaPlan plan;
  plan.total_units = (a.n + 31) / 32;
  plan.ctas = plan.total_units < sm_count() ? plan.total_units : sm_count();
  plan.smax = 1;
  for (int cta = 0; cta < plan.ctas; ++cta) {  // a CTA's strips: whole ones of four units, then the rest
    const int units = static_cast<int>(static_cast<int64_t>(cta + 1) * plan.total_units / plan.ctas - static_cast<int64_t>(cta) * plan.total_units / plan.ctas);
    if (units % 4 != 0) plan.smax = max(plan.smax, umma_split(units % 4, a.k, kUStepK));
  }
  plan.xdepth = 8 / plan.smax < kUMaxXBufs ? 8 / plan.smax : kUMaxXBufs;
  plan.stages = plan.smax <= 2 ? kUMaxStages : 2;  // 16 smax accumulator columns per issuer must fit beside the stages
  const size_t smem = kUPackedBufs * kUPackedBytes + 2 * kUXRegion + 128 * a.groups * 2 + kURedBytes + 48 * sizeof(uint64_t);
  if (smem > 225 * 1024) return XDK_ERR_LIMIT;
  CUtensorMap wmap, smap, xmap;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.k / 8), static_cast<cuuint64_t>(a.n)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.k / 2)};
    const cuuint32_t box[2] = {kUStepK / 8, 32};
    const cuuint64_t sdims[2] = {static_cast<cuuint64_t>(a.groups), static_cast<cuuint64_t>(a.n)};
    const cuuint64_t sstrides[1] = {static_cast<cuuint64_t>(a.groups) * 2};
    const cuuint32_t sbox[2] = {static_cast<cuuint32_t>(a.groups), 32};
    static_assert(kUStepK / 2 == 128, "the packed box is one 128-byte swizzle span wide");
    if (!encode_tiled(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, a.packed, dims, strides, box, true) ||
        !encode_tiled(&smap, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, a.scales, sdims, sstrides, sbox, false))
      return XDK_ERR_LAUNCH;
    const cuuint64_t xdims[2] = {static_cast<cuuint64_t>(a.k), static_cast<cuuint64_t>(a.m)};
    const cuuint64_t xstrides[1] = {static_cast<cuuint64_t>(a.k) * 2};
    const cuuint32_t xbox[2] = {kUStepK, 16};
    if (!encode_tiled(&xmap, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, a.x, xdims, xstrides, xbox, false)) return XDK_ERR_LAUNCH;
  }
  cudaError_t err = cudaFuncSetAttribute(w4a16_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (err != cudaSuccess) return note_launch(err);
  return launch_opts(w4a16_umma_kernel, dim3(plan.ctas), dim3(kUThreads), smem, stream, 1u, dependent, a, plan, wmap, smap, xmap);
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

// ------------------------------------------------------------------------------------------------
// Direct-load tensor-core path for M <= 8 and K % 1024 == 0.
//
// The SIMT kernel spends five thread instructions per code (the exact unpack, then an FMA per code and row with
// both operands taken out of their half2 pairs) and is issue-bound at a third of the HBM rate on this part.  Here
// the unpack's half2 pairs go to mma.m16n8k16 as they are, with the operands swapped so that no row of the MMA is
// wasted on small M: the 16 rows of the MMA are 16 columns of W, its 8 columns are the (up to 8) rows of x.  Lane
// (n = lane / 4, q = lane % 4) loads the 16-byte vectors (32 codes) of columns n and n + 8 that start at
// k = chunk + 32 q.  An MMA does not care which k a fragment slot stands for as long as A and B agree, so slot pairs
// are simply "the pairs the unpack produces": word w of a vector gives A pairs (k0,k4) (k1,k5) for one MMA and
// (k2,k6) (k3,k7) for the next, and the matching B pairs are one 16-byte read of x, which sits in shared memory
// already permuted to (0,4,1,5,2,6,3,7) inside every 8 k.  The legacy HMMA pipe of this part retires one m16n8k16
// per 32 cycles and sub-partition (6.3 us for K = 4096, N = 14336 in this form; with x as the 16-row operand it
// would be twice that), so the rest of the instruction stream has to fit beside it: 26 warp instructions per MMA
// are left (13 of them the exact unpack), after taking everything out of the loop that does not depend on the
// codes -- no zero-filling of registers for columns past N or rows past M (they read a valid column or row and
// feed outputs that are never stored), scales widened to half2 when they are fetched, one base pointer per column.
// The grid is one wave (as many CTAs as are resident at once), the groups of 16 columns dealt evenly.
// A CTA is eight warps that split K eight ways over the same 16 columns and add their partial sums in shared
// memory in warp order.  A warp's work is a sequence of batches (a column pass x a round of up to four 128-k chunks
// of its K share); the loads of the next batch are in flight while the current one is unpacked and multiplied, in
// two register buffers, so the weight stream never waits for the tensor pipe nor the pipe for the stream.
struct MmaBatch {
  U4 wv[4][2];      // [chunk][column n, column n + 8]: 32 codes each
  __half2 sc[4][2]; // their scale, in both halves
};

__global__ void __launch_bounds__(kThreads, 2)
w4a16_mma_kernel(W4Args a, int col_groups) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int pitch = a.k * 2 + 16;                          // bytes per x row: the pad puts the 8 rows on different banks
  unsigned char* xs = smem_raw;                            // [m rows][pitch], k permuted inside every 8
  float* red = reinterpret_cast<float*>(smem_raw + ((static_cast<size_t>(a.m) * pitch + 127) & ~static_cast<size_t>(127)));  // [2][8 warps][32 lanes][4]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = lane >> 2, q = lane & 3;
  const int row_bytes = a.k / 2;
  const int k_warp = a.k / kWarps;          // this warp's share of K, a multiple of 128
  const int chunks = k_warp / 128;          // 128 k per chunk: 32 per lane of a quad
  constexpr int kBatchChunks = 4;
  const int rounds = (chunks + kBatchChunks - 1) / kBatchChunks;
  const int k0 = warp * k_warp + q * 32;    // first k of this lane's vectors
  // the groups of 16 columns are dealt evenly to the CTAs of the grid (all resident at once: no second wave)
  const int group0 = static_cast<int>(static_cast<int64_t>(blockIdx.x) * col_groups / gridDim.x);
  const int my_passes = static_cast<int>(static_cast<int64_t>(blockIdx.x + 1) * col_groups / gridDim.x) - group0;  // >= 1
  const int cta_col0 = group0 * 16;

  const int scale_shift = 31 - __clz(a.group);  // group sizes are powers of two
  // Columns past N (the last pass of the last CTA when N % 16 != 0) read the last column instead and chunks past the
  // warp's share are not loaded at all: what they would feed is never stored, respectively never computed.
  auto fetch = [&](MmaBatch& b, int col_base, int chunk0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int col = min(col_base + h * 8 + n, a.n - 1), k = k0 + chunk0 * 128;
      const uint8_t* wp = a.packed + static_cast<size_t>(col) * row_bytes + k / 2;
      const __half* sp = a.scales + static_cast<size_t>(col) * a.groups;
#pragma unroll
      for (int c = 0; c < kBatchChunks; ++c)
        if (chunk0 + c < chunks) {
          b.wv[c][h] = ld_stream16(wp + c * 64);
          b.sc[c][h] = __half2half2(__ldg(sp + ((k + c * 128) >> scale_shift)));
        }
    }
  };
  MmaBatch buf0, buf1;
  pdl_launch_dependents();
  fetch(buf0, cta_col0, 0);  // the first batch's weights go out before x is staged
  pdl_wait();                // x may be the preceding kernel's output; the weights are not

  const int units = a.k / 8;
  for (int i = threadIdx.x; i < a.m * units; i += kThreads) {
    const int r = i / units, u = i - r * units;
    const U4 v = ld_cached16(a.x + static_cast<size_t>(r) * a.k + u * 8);
    U4 o;  // k 0..7 -> 0,4,1,5,2,6,3,7: the pairs the unpack produces
    o.x = __byte_perm(v.x, v.z, 0x5410);
    o.y = __byte_perm(v.x, v.z, 0x7632);
    o.z = __byte_perm(v.y, v.w, 0x5410);
    o.w = __byte_perm(v.y, v.w, 0x7632);
    *reinterpret_cast<U4*>(xs + static_cast<size_t>(r) * pitch + u * 16) = o;
  }
  __syncthreads();
  // this lane's B fragments: row n of x; lanes past M read row 0 and feed output rows that are never stored
  const unsigned char* xrow = xs + static_cast<size_t>(n < a.m ? n : 0) * pitch;

  // two accumulator sets (the two MMAs of a word alternate, halving the dependent chain), summed at the end of a pass:
  // (column n, rows 2 q + {0, 1} of x), (column n + 8, the same rows)
  float acc0[4], acc1[4];
  int pass = 0, round = 0;  // of the batch being computed
  auto step = [&](MmaBatch& cur, MmaBatch& nxt) -> bool {
    int np = pass, nr = round + 1;
    if (nr == rounds) nr = 0, ++np;
    const bool has_next = np < my_passes;
    if (has_next) fetch(nxt, cta_col0 + np * 16, nr * kBatchChunks);
    if (round == 0) {
#pragma unroll
      for (int e = 0; e < 4; ++e) acc0[e] = acc1[e] = 0.0f;
    }
    const int chunk0 = round * kBatchChunks;
#pragma unroll
    for (int c = 0; c < kBatchChunks; ++c) {
      if (chunk0 + c < chunks) {
        const unsigned char* xk = xrow + (k0 + (chunk0 + c) * 128) * 2;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const U4 xv = *reinterpret_cast<const U4*>(xk + w * 16);
          const uint32_t w0 = w == 0 ? cur.wv[c][0].x : (w == 1 ? cur.wv[c][0].y : (w == 2 ? cur.wv[c][0].z : cur.wv[c][0].w));
          const uint32_t w1 = w == 0 ? cur.wv[c][1].x : (w == 1 ? cur.wv[c][1].y : (w == 2 ? cur.wv[c][1].z : cur.wv[c][1].w));
          __half2 h0[4], h1[4];
          dequant8(w0, cur.sc[c][0], h0);
          dequant8(w1, cur.sc[c][1], h1);
          mma16816(acc0, *reinterpret_cast<uint32_t*>(&h0[0]), *reinterpret_cast<uint32_t*>(&h1[0]), *reinterpret_cast<uint32_t*>(&h0[1]),
                   *reinterpret_cast<uint32_t*>(&h1[1]), xv.x, xv.y);
          mma16816(acc1, *reinterpret_cast<uint32_t*>(&h0[2]), *reinterpret_cast<uint32_t*>(&h1[2]), *reinterpret_cast<uint32_t*>(&h0[3]),
                   *reinterpret_cast<uint32_t*>(&h1[3]), xv.z, xv.w);
        }
      }
    }
    if (round == rounds - 1) {
      // the partial sums of the pass meet in shared memory; the buffer alternates between passes, so one barrier
      // per pass is enough (the warp that adds pass p has passed the barrier of pass p + 1 before anybody writes
      // the buffer of pass p + 2), and the adding warp rotates
      float* mine = red + (pass & 1) * (kWarps * 32 * 4);
      *reinterpret_cast<float4*>(mine + (warp * 32 + lane) * 4) =
          make_float4(__fadd_rn(acc0[0], acc1[0]), __fadd_rn(acc0[1], acc1[1]), __fadd_rn(acc0[2], acc1[2]), __fadd_rn(acc0[3], acc1[3]));
      __syncthreads();
      if (warp == (pass & (kWarps - 1))) {  // the eight partial sums in warp order, bias, store
        const int col_base = cta_col0 + pass * 16;
        float4 total = *reinterpret_cast<const float4*>(mine + lane * 4);
        for (int w = 1; w < kWarps; ++w) {
          const float4 part = *reinterpret_cast<const float4*>(mine + (w * 32 + lane) * 4);
          total.x = __fadd_rn(total.x, part.x), total.y = __fadd_rn(total.y, part.y);
          total.z = __fadd_rn(total.z, part.z), total.w = __fadd_rn(total.w, part.w);
        }
        const float out[4] = {total.x, total.y, total.z, total.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = col_base + (e >> 1) * 8 + n, row = q * 2 + (e & 1);
          if (row < a.m && col < a.n)
            a.y[static_cast<size_t>(row) * a.n + col] = __float2half_rn(out[e] + (a.bias ? __half2float(a.bias[col]) : 0.0f));
        }
      }
    }
    pass = np, round = nr;
    return has_next;
  };
  while (step(buf0, buf1) && step(buf1, buf0)) {
  }
}

int launch_mma(W4Args a, bool dependent, cudaStream_t stream) {
  const size_t xbytes = (static_cast<size_t>(a.m) * (a.k * 2 + 16) + 127) & ~static_cast<size_t>(127);
  const size_t smem = xbytes + 2 * static_cast<size_t>(kWarps) * 32 * 4 * sizeof(float);
  cudaError_t err = cudaFuncSetAttribute(w4a16_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (err != cudaSuccess) return note_launch(err);
  // one wave: as many CTAs as the device holds at once (two per SM unless x takes more than half the shared memory);
  // a grid of a few CTAs more than that ran as two waves and took twice the time
  int resident = 0;
  err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, w4a16_mma_kernel, kThreads, smem);
  if (err != cudaSuccess) return note_launch(err);
  if (resident < 1) return XDK_ERR_LIMIT;
  const int groups = (a.n + 15) / 16;
  const int ctas = groups < resident * sm_count() ? groups : resident * sm_count();
  return launch_opts(w4a16_mma_kernel, dim3(ctas), dim3(kThreads), smem, stream, 1u, dependent, a, groups);
}

template <int MT, int CW>
int launch_simt(W4Args a, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(MT) * a.k * sizeof(__half);
  auto kernel = w4a16_simt_kernel<MT, CW>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (err != cudaSuccess) return note_launch(err);
  a.col_groups = (a.n + kWarps * CW - 1) / (kWarps * CW);
  const int max_ctas = 4 * sm_count();
  a.groups_per_cta = (a.col_groups + max_ctas - 1) / max_ctas;
  const int ctas = (a.col_groups + a.groups_per_cta - 1) / a.groups_per_cta;
  return launch(kernel, dim3(ctas), dim3(kThreads), smem, stream, 1u, a);
}

}  // namespace
}  // namespace xdk

namespace xdk {
unsigned w4a16_fault_word() {
  unsigned v = 0;
  if (cudaMemcpyFromSymbol(&v, g_w4_fault, sizeof(v)) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0x80000000u;
  }
  return v;
}
}  // namespace xdk

extern "C" int xdk_w4a16(const void* x, const uint8_t* packed, const void* scales, const void* bias, void* y,
                         int64_t m, int64_t k, int64_t n, int group_size, void* stream) {
  return xdk_w4a16_v2(x, packed, scales, bias, y, m, k, n, group_size, 0u, stream);
}

extern "C" int xdk_w4a16_v2(const void* x, const uint8_t* packed, const void* scales, const void* bias, void* y,
                            int64_t m, int64_t k, int64_t n, int group_size, unsigned flags, void* stream) {
  if (!y || n < 1) return XDK_ERR_ARG;
  xdk_peer_out one = {};
  one.ptr[0] = y, one.world = 1, one.ld = n, one.col0 = 0;
  return xdk_w4a16_peer(x, packed, scales, bias, &one, m, k, n, group_size, flags, stream);
}

extern "C" int xdk_w4a16_peer(const void* x, const uint8_t* packed, const void* scales, const void* bias,
                              const xdk_peer_out* y_out, int64_t m, int64_t k, int64_t n, int group_size, unsigned flags,
                              void* stream) {
  using namespace xdk;
  if (flags & ~XDK_DEPENDENT_LAUNCH) return XDK_ERR_ARG;
  PeerOut out;
  if (int st = make_out(y_out, nullptr, n, &out)) return st;
  void* y = out.ptr[0];
  const bool plain = out.world == 1 && out.ld == n && out.col0 == 0;  // the kernels of this file write y[m][n] only
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
  const bool dependent = (flags & XDK_DEPENDENT_LAUNCH) != 0;
  a.out = out;
  const bool vec_ok = k % 32 == 0 && aligned16(packed) && aligned16(x);  // 16-byte vectors of 32 codes
  // M <= 8 with K a multiple of 1024 and x small enough for shared memory: the direct-load mma.sync kernel
  // (K = 4096: N = 4096 5.9 / 6.0 / 6.4 / 7.2 us at M = 1 / 2 / 4 / 8, N = 14336 14.7 / 14.8 / 15.3 / 16.1, N = 28672
  // 23.3 - 24.9; K = 14336, N = 4096: 13.9 / 14.6 / 19.9 at M = 1 / 2 / 4 -- against 6.4 / 16.3 / 30.1 / 17.3 at M = 1
  // for the SIMT kernel and 10.2 - 10.8 / 16.6 - 17.0 / 28.5 - 29.2 / 21.5 - 25.8 for the tcgen05 kernel).
  // XDK_W4A16_MMA=0 leaves these shapes to the kernels below (comparison runs).
  static const bool mma_env = !(getenv("XDK_W4A16_MMA") && getenv("XDK_W4A16_MMA")[0] == '0');
  if (mma_env && plain && vec_ok && m <= 8 && k % 1024 == 0 &&
      static_cast<size_t>(m) * (static_cast<size_t>(k) * 2 + 16) <= 160 * 1024)
    return launch_mma(a, dependent, s);
  // M >= 9, smaller M where the kernel above does not apply (M >= 3, M = 2 on large matrices), and every M whose
  // output is strided or goes to several ranks: the tcgen05 kernel.  Its time hardly depends on M (K = 4096,
  // N = 14336: 17.1 us at M = 1, 17.6 at M = 8, 18.2 at M = 16).  XDK_W4A16_UMMA=0 keeps it for strided and
  // multi-rank outputs only (comparison runs).
  static const int umma_env = getenv("XDK_W4A16_UMMA") ? (getenv("XDK_W4A16_UMMA")[0] == '1' ? 1 : 0) : -1;
  const bool umma_ok = vec_ok && k % 256 == 0 && group_size >= 64 && a.groups <= 256 && a.groups % 8 == 0 && aligned16(scales);
  const int umma_min_m = k * n >= (32LL << 20) ? 2 : 3;
  if (umma_ok && ((umma_env != 0 && m >= umma_min_m) || !plain)) {
    const int st = launch_umma(a, dependent, s);
    if (st != XDK_ERR_LIMIT || !plain) return st;
  }
  if (!plain) return XDK_ERR_LIMIT;  // a strided or multi-rank destination needs the tcgen05 kernel's shape
  if (vec_ok && k % 128 == 0 && m >= 3) return m > 8 ? launch_stream<16>(a, s) : launch_stream<8>(a, s);
  // the SIMT kernel keeps all rows of x (padded to a power of two) in shared memory
  const int mt = m == 1 ? 1 : (m == 2 ? 2 : (m <= 4 ? 4 : (m <= 8 ? 8 : 16)));
  if (vec_ok && static_cast<int64_t>(mt) * k * 2 <= 200 * 1024) {
    if (mt == 1) return launch_simt<1, 2>(a, s);
    if (mt == 2) return launch_simt<2, 2>(a, s);
    if (mt == 4) return launch_simt<4, 2>(a, s);
    if (mt == 8) return launch_simt<8, 1>(a, s);
    return launch_simt<16, 1>(a, s);
  }
  return launch(w4a16_generic_kernel, dim3(static_cast<unsigned>((n + kWarps - 1) / kWarps)), dim3(kThreads), 0, s, 1u,
                a);
}
