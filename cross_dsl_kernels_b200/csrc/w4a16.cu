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
// Two compute paths share the unpack:
//   * M <= 2: SIMT.  Lanes stride over the packed row, weights feed mixed-precision FMAs
//     (FP16 operands, FP32 accumulator) and a warp shuffle finishes each column.
//   * 3 <= M <= 16: tensor cores.  The op is then a real [16 x K] x [K x N] contraction: x is padded to
//     16 rows and the dequantised weights go straight from registers into mma.m16n8k16 B fragments
//     (FP32 accumulators).  The k order inside a fragment is free as long as A uses the same order, so
//     x is stored in shared memory pre-permuted to the order the unpack produces and no weight ever
//     moves between lanes.
// Split-K slices of one column strip form a thread-block cluster and are summed in slice order
// through distributed shared memory (one launch, no scratch, deterministic).
#include <cooperative_groups.h>
#include <stdlib.h>

#include "common.cuh"

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

// One TMA op: the 2-D box at element coordinates (c0, c1) of `map` -> dense rows at dst; completes on `bar`.
__device__ __forceinline__ void tma_box_2d(void* dst_smem, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst_smem)),
      "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}

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
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      sm_count = 148;
  }
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
    if (!encode_tiled_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, a.packed, dims, strides, box, false)) return XDK_ERR_LAUNCH;
    smap = wmap;
    if (plan.ring_scales) {
      const cuuint64_t sdims[2] = {static_cast<cuuint64_t>(a.groups), static_cast<cuuint64_t>(a.n)};
      const cuuint64_t sstrides[1] = {static_cast<cuuint64_t>(a.groups) * 2};
      const cuuint32_t sbox[2] = {static_cast<cuuint32_t>(kChunkK / a.group), 8};
      if (!encode_tiled_2d(&smap, CU_TENSOR_MAP_DATA_TYPE_UINT16, a.scales, sdims, sstrides, sbox, false)) return XDK_ERR_LAUNCH;
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
        n = sm_count;
      } else {
        cfg.gridDim = dim3(sm_count / sz * sz);
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
    if (fit * sz * 100 < sm_count * 94) continue;
    const int clusters = min(fit, plan.total_blocks);
    if ((plan.total_blocks + clusters - 1) / clusters > kStreamWarps * kMaxNB) continue;
    best_log2 = s_log2;
    break;
  }
  plan.splits = 1 << best_log2;
  plan.clusters = min(resident_clusters(best_log2), plan.total_blocks);
  if (plan.clusters <= 0) plan.clusters = min(sm_count, plan.total_blocks), plan.splits = 1;
  cfg.gridDim = dim3(plan.clusters * plan.splits);
  attr[0].val.clusterDim.x = plan.splits;
  cfg.numAttrs = plan.splits > 1 ? 1 : 0;
  return note_launch(cudaLaunchKernelEx(&cfg, kernel, a, plan, wmap, smap));
}


// ------------------------------------------------------------------------------------------------
// tcgen05 path (M > 8, K % 256 == 0, group >= 64): the contraction runs on the 5th-generation tensor
// cores.  Operands are swapped so that the UMMA "M" dimension is a strip of up to 128 output columns:
//     D[128 columns x 16 tokens] += A[128 x 16 k] * B[16 k x 16],   A = dequantised W,  B = x^T
// and A lives in TENSOR MEMORY: the unpack warps write the dequantised weights straight from registers
// into TMEM (tcgen05.st), so they never pass through shared memory.  (With A in shared memory every
// M=128,N=16 MMA re-reads 4 KB of A for 16 columns of use, which by itself saturates the 128 B/clk
// shared-memory port and starves the unpack warps that share it.)
// One persistent CTA per SM owns a contiguous, evenly dealt range of 8-column blocks and walks it
// in strips of <= 128 columns, full K each (no split-K, no cross-CTA reduction).
//   warp 8, one lane : TMA box copies of the packed codes of a (strip, 256-k chunk) -- one 4 KB box per
//                      32 columns, 128-byte swizzled -- into a ring of chunk buffers, plus the strip's scales
//   warps 10-11      : stage x for each chunk in shared memory (k order of the unpack, canonical K-major
//                      core-matrix layout); x is the B operand, read through a shared-memory descriptor
//   warps 0-7        : thread = one column of the strip (TMEM lane); warp w owns lane quarter w % 4 and k half
//                      w / 4 of every 256-k stage (= chunk): 16-byte shared loads of codes -> dequant -> tcgen05.st
//   warps 9, 12-14   : MMA issuers, one lane each.  A warp gets a tcgen05.mma out only every ~100 cycles, whatever
//                      the shape (measured: 94-118 cycles per M=128 MMA for N = 16 .. 128), while four warps
//                      issuing side by side reach one per ~29 cycles.  So the 8 K=16 blocks of a stage are dealt
//                      round-robin to 4 issuers, each accumulating into its OWN 128 x 16 FP32 accumulator, then
//                      tcgen05.commit onto the barriers (count 4) that hand the stage / x buffer back and
//                      announce the finished strip
//   warps 0-3        : epilogue -- tcgen05.ld of the four accumulators, summed in fixed order, bias, FP16 store
// TMEM columns (512 allocated; the kernel is alone on its SM): 16 i .. accumulator of issuer i, 64 + 64 s .. A stage s.
// Every wait is time-bounded; on a timeout the kernel raises g_w4_fault, stops issuing work, and still
// frees its TMEM columns before it returns.
constexpr int kUChunkK = 256;                  // k per packed chunk
constexpr int kUPackedBufs = 8;                // packed chunks in flight (16 KB each at 128 columns)
constexpr int kUStageK = 256;                  // k per unpack/MMA stage (= one packed chunk: fewer hand-offs per k)
constexpr int kUStages = 3;                    // A operand stages in TMEM
constexpr int kUTmemCols = 512;                // allocation (power of two)
constexpr int kUTmemA = 64;                    // first column of A stage 0
constexpr int kUStageCols = kUStageK / 2;      // 32-bit TMEM columns per stage (two FP16 k per column)
static_assert(kUTmemA + kUStages * kUStageCols <= kUTmemCols, "A stages must fit the TMEM allocation");
constexpr int kUXLbo = 128, kUXSbo = (kUChunkK / 8) * kUXLbo;  // x chunk: [2 row groups][32 k groups][8 x 16 B]
constexpr int kUXBytes = 2 * kUXSbo;
constexpr int kUPackedBytes = 16 * 8 * (kUChunkK / 2);  // packed codes of a 128-column strip chunk
constexpr int kUIssuers = 4;                   // MMA-issuing warps, one accumulator each
constexpr int kUThreads = 15 * 32;             // 8 unpack warps, TMA warp, MMA warp 0, 2 x-staging warps, MMA warps 1-3

struct UmmaPlan {
  int ctas, total_blocks, chunks;  // total_blocks counts 32-column units
  int scale_row_bytes;  // bytes of scales per column (groups * 2)
};

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, int lbo, int sbo) {
  return static_cast<uint64_t>((smem_addr >> 4) & 0x3fff) | (static_cast<uint64_t>((lbo >> 4) & 0x3fff) << 16) |
         (static_cast<uint64_t>((sbo >> 4) & 0x3fff) << 32) | (1ull << 46);  // version 1, no swizzle
}
// D (TMEM) (+)= A (TMEM) * B (shared memory descriptor)
__device__ __forceinline__ void umma_f16_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_cta(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(kUThreads, 1)
w4a16_umma_kernel(W4Args a, UmmaPlan plan, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* packed = smem_raw;                                   // [kUPackedBufs][kUPackedBytes]
  unsigned char* xbuf = packed + kUPackedBufs * kUPackedBytes;        // [2][kUXBytes]
  unsigned char* scbuf = xbuf + 2 * kUXBytes;                         // [16 blocks][8 cols][scale_row_bytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(scbuf + 16 * 8 * plan.scale_row_bytes);
  uint64_t* pk_full = bars;                       // [kUPackedBufs]  TMA bytes of a packed chunk landed
  uint64_t* pk_empty = bars + kUPackedBufs;       // [kUPackedBufs]  the 8 unpack warps are done with the chunk
  uint64_t* a_full = bars + 2 * kUPackedBufs;     // [kUStages] the 8 unpack warps wrote the stage to TMEM
  uint64_t* a_empty = a_full + kUStages;          // [kUStages] MMAs that read the stage completed (commit)
  uint64_t* x_full = a_empty + kUStages;          // [2]
  uint64_t* x_empty = x_full + 2;                // [2]
  uint64_t* sc_full = x_empty + 2;               // [1]
  uint64_t* acc_full = sc_full + 1;              // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the CTA's range of 8-column blocks, dealt in units of 4 blocks (one TMEM lane quarter, one 32-row TMA box)
  const int blk_begin = 4 * static_cast<int>(static_cast<int64_t>(blockIdx.x) * plan.total_blocks / plan.ctas);
  const int blk_end = 4 * static_cast<int>(static_cast<int64_t>(blockIdx.x + 1) * plan.total_blocks / plan.ctas);
  const int scale_shift = 31 - __clz(a.group);

  if (threadIdx.x == 0) {
    for (int i = 0; i < kUPackedBufs; ++i) {
      mbar_init(pk_full + i, 1);
      mbar_init(pk_empty + i, 8);   // one arrival per unpack warp
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(x_full + i, 2);   // one arrival per x-staging warp
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
  if (warp == 9) {  // TMEM: accumulator + A stages
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(kUTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;

  if (warp == 8) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int q = 0, strip_i = 0;  // chunk counter over the CTA's life, strip counter
      bool ok = true;
      for (int b0 = blk_begin; b0 < blk_end && ok; b0 += 16, ++strip_i) {
        const int nb = min(16, blk_end - b0);
        // scales of the strip (whole K): wait until the previous strip's readers are done = its last chunk buffer was released
        if (strip_i > 0) {
          const int prev = q - 1;  // last chunk of the previous strip
          ok = mbar_wait(pk_empty + prev % kUPackedBufs, (prev / kUPackedBufs) & 1);
          if (!ok) break;
        }
        mbar_expect_tx(sc_full, static_cast<unsigned>(nb * 8 * plan.scale_row_bytes));
        for (int b = 0; b < nb; b += 4) tma_box_2d(scbuf + b * 8 * plan.scale_row_bytes, &smap, 0, (b0 + b) * 8, sc_full);
        for (int kc = 0; kc < plan.chunks; ++kc, ++q) {
          const int buf = q % kUPackedBufs;
          if (q >= kUPackedBufs && !mbar_wait(pk_empty + buf, ((q / kUPackedBufs) - 1) & 1)) {
            ok = false;
            break;
          }
          mbar_expect_tx(pk_full + buf, static_cast<unsigned>(nb * 8 * (kUChunkK / 2)));
          for (int b = 0; b < nb; b += 4)  // 32-row boxes; the 128-byte swizzle depends on (row & 7) only, so rows stay where 8-row boxes put them
            tma_box_2d(packed + buf * kUPackedBytes + b * 8 * (kUChunkK / 2), &wmap, kc * (kUChunkK / 8), (b0 + b) * 8, pk_full + buf);
        }
      }
      if (!ok) atomicOr(&g_w4_fault, 4u);
    }
  } else if (warp == 9 || warp >= 12) {
    // ------------------------------------------------------------ MMA issuers
    if (lane == 0) {
      constexpr uint32_t kIdesc = (1u << 4) | (2u << 17) | (8u << 24);  // D = F32, A = B = F16 K-major, N = 16, M = 128
      const int issuer = warp == 9 ? 0 : warp - 11;
      const uint32_t acc = tmem_acc + issuer * 16;
      // x descriptor: only the 14-bit start-address field changes from MMA to MMA
      const uint64_t xd0 = umma_desc(smem_u32(xbuf), kUXLbo, kUXSbo);
      const uint32_t xd_lo = static_cast<uint32_t>(xd0), xd_hi = static_cast<uint32_t>(xd0 >> 32);
      int q = 0, sq = 0;  // chunk counter, stage counter
      bool ok = true;
      for (int b0 = blk_begin; b0 < blk_end && ok; b0 += 16) {
        for (int kc = 0; kc < plan.chunks && ok; ++kc, ++q) {
          const int xb = q & 1;
          ok = mbar_wait(x_full + xb, (q >> 1) & 1);
          for (int st = 0; st < kUChunkK / kUStageK && ok; ++st, ++sq) {
            const int s = sq % kUStages;
            ok = mbar_wait(a_full + s, (sq / kUStages) & 1);
            if (!ok) break;
            tc_fence_after();
            const uint32_t a_base = tmem_acc + kUTmemA + s * kUStageCols + issuer * 8;
            const uint32_t x_lo = xd_lo + ((xb * kUXBytes + (st * (kUStageK / 8) + issuer * 2) * kUXLbo) >> 4);
#pragma unroll
            for (int j = 0; j < kUStageK / 16 / kUIssuers; ++j) {  // K blocks issuer, issuer + 4, ...
              uint64_t xd;
              asm("mov.b64 %0, {%1, %2};" : "=l"(xd) : "r"(x_lo + ((j * kUIssuers * 2 * kUXLbo) >> 4)), "r"(xd_hi));
              umma_f16_ta(acc, a_base + j * kUIssuers * 8, xd, kIdesc, !(kc == 0 && st == 0 && j == 0));
            }
            umma_commit(a_empty + s);  // the TMEM stage is free once every issuer's MMAs have read it
          }
          if (ok) umma_commit(x_empty + xb);
        }
        if (ok) umma_commit(acc_full);
      }
      if (!ok) atomicOr(&g_w4_fault, 8u);
    }
  } else if (warp >= 10) {  // 10, 11
    // ------------------------------------------------------------ x staging warps
    // x chunk -> canonical K-major layout with the unpack's k order inside each 8-block.  The global loads
    // of a chunk are issued one chunk ahead, so only the permute + stores sit between two hand-offs.
    const int t = threadIdx.x - 320;  // 0 .. 63
    U4 xin[8];
    auto load_x = [&](int kc) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = t + i * 64;  // 16 rows x 32 k groups; a warp covers 8 rows x 4 k groups = 512 contiguous bytes of xbuf
        const int m = (idx & 7) | ((idx >> 8) << 3), kg = (idx >> 3) & 31;
        xin[i] = U4{0u, 0u, 0u, 0u};
        if (m < a.m) xin[i] = ld_cached16(a.x + static_cast<size_t>(m) * a.k + kc * kUChunkK + kg * 8);
      }
    };
    load_x(0);
    int q = 0;
    bool ok = true;
    for (int b0 = blk_begin; b0 < blk_end; b0 += 16) {
      for (int kc = 0; kc < plan.chunks; ++kc, ++q) {
        const int xb = q & 1;
        if (ok && q >= 2) ok = mbar_wait(x_empty + xb, ((q >> 1) - 1) & 1);
        if (ok) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int idx = t + i * 64;
            const int m = (idx & 7) | ((idx >> 8) << 3), kg = (idx >> 3) & 31;
            U4 v;
            v.x = __byte_perm(xin[i].x, xin[i].z, 0x5410);
            v.y = __byte_perm(xin[i].x, xin[i].z, 0x7632);
            v.z = __byte_perm(xin[i].y, xin[i].w, 0x5410);
            v.w = __byte_perm(xin[i].y, xin[i].w, 0x7632);
            *reinterpret_cast<U4*>(xbuf + xb * kUXBytes + (m >> 3) * kUXSbo + kg * kUXLbo + (m & 7) * 16) = v;
          }
          fence_async_smem();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_cta(x_full + xb);
        load_x(kc + 1 < plan.chunks ? kc + 1 : 0);  // next chunk (x does not depend on the strip)
      }
    }
    if (!ok && lane == 0) atomicOr(&g_w4_fault, 32u);
  } else {
    // ------------------------------------------------------------ unpack warps (+ epilogue)
    const int lq = warp & 3, kh = warp >> 2;  // TMEM lane quarter this warp may touch, k half of a stage
    const int c = lq * 32 + lane;             // this thread's column of the strip = its TMEM lane
    const uint32_t a_lane_base = tmem_acc + (static_cast<uint32_t>(lq * 32) << 16) + kUTmemA + kh * (kUStageCols / 2);
    int q = 0, sq = 0, strip_i = 0;
    bool ok = true;
    for (int b0 = blk_begin; b0 < blk_end; b0 += 16, ++strip_i) {
      const int nb = min(16, blk_end - b0);
      const int ncols = nb * 8;
      const bool warp_live = lq * 32 < ncols;  // warp-uniform: a quarter without columns writes nothing
      if (ok) ok = mbar_wait(sc_full, strip_i & 1);
      const unsigned char* sc_row = scbuf + c * plan.scale_row_bytes;
      for (int kc = 0; kc < plan.chunks; ++kc, ++q) {
        const int buf = q % kUPackedBufs;
        if (ok) ok = mbar_wait(pk_full + buf, (q / kUPackedBufs) & 1);
        // packed tiles arrive 128-byte swizzled: 16-byte piece p of row r sits at piece p ^ (r & 7), so the
        // lanes of a warp, which read the same piece of 32 different rows, spread over all bank groups
        const unsigned char* row = packed + buf * kUPackedBytes + (c >> 3) * 8 * (kUChunkK / 2) + (c & 7) * (kUChunkK / 2);
        for (int st = 0; st < kUChunkK / kUStageK; ++st, ++sq) {
          const int s = sq % kUStages;
          if (ok && sq >= kUStages) ok = mbar_wait(a_empty + s, ((sq / kUStages) - 1) & 1);
          if (ok && warp_live) {
            tc_fence_after();
            const int k_half = kc * kUChunkK + st * kUStageK + kh * (kUStageK / 2);
#pragma unroll
            for (int pc = 0; pc < kUStageK / 64; ++pc) {
              // two pieces = 64 k lie inside one group (group >= 64)
              const __half2 s2 = __half2half2(reinterpret_cast<const __half*>(sc_row)[(k_half + (pc & ~1) * 32) >> scale_shift]);
              const int piece = st * (kUStageK / 32) + kh * (kUStageK / 64) + pc;
              U4 wv = U4{0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u};  // code 8 = weight 0 for columns past the strip
              if (c < ncols) wv = *reinterpret_cast<const U4*>(row + ((piece ^ (c & 7)) << 4));
              uint32_t r[16];
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                const uint32_t word = w == 0 ? wv.x : (w == 1 ? wv.y : (w == 2 ? wv.z : wv.w));
                __half2 h[4];
                dequant8(word, s2, h);
#pragma unroll
                for (int i = 0; i < 4; ++i) r[4 * w + i] = *reinterpret_cast<uint32_t*>(&h[i]);
              }
              tmem_st16(a_lane_base + s * kUStageCols + pc * 16, r);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
          }
          __syncwarp();
          if (lane == 0) mbar_arrive_cta(a_full + s);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_cta(pk_empty + buf);
      }
      // ---- epilogue of the strip: warps 0-3 read TMEM lanes 32*warp .. +31 = columns of the strip
      if (warp < 4) {
        if (ok) ok = mbar_wait(acc_full, strip_i & 1);
        if (ok) {
          tc_fence_after();
          float sum[16];
          const uint32_t taddr = tmem_acc + (static_cast<uint32_t>(warp * 32) << 16);
#pragma unroll
          for (int i = 0; i < kUIssuers; ++i) {
            uint32_t r[16];
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                  "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                : "r"(taddr + i * 16));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int m = 0; m < 16; ++m) sum[m] = i == 0 ? __uint_as_float(r[m]) : __fadd_rn(sum[m], __uint_as_float(r[m]));
          }
          const int col = b0 * 8 + c;  // warps 0-3: lq == warp, so c is this thread's accumulator lane too
          if (c < ncols && col < a.n) {
            const float bv = a.bias ? __half2float(a.bias[col]) : 0.0f;
#pragma unroll
            for (int m = 0; m < 16; ++m)
              if (m < a.m) a.y[static_cast<size_t>(m) * a.n + col] = __float2half_rn(sum[m] + bv);
          }
          tc_fence_before();
        }
      }
      // all 256 threads meet before the next strip's stages can reach the MMA warp (its a_full needs all of them),
      // so the next strip's first MMA cannot overwrite TMEM while it is still being read
      asm volatile("bar.sync 1, 256;" ::: "memory");
    }
    if (!ok && lane == 0) atomicOr(&g_w4_fault, 16u);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "n"(kUTmemCols) : "memory");
  }
}

int launch_umma(const W4Args& a, cudaStream_t stream) {
  UmmaPlan plan;
  plan.total_blocks = (a.n + 31) / 32;  // units of 32 columns
  plan.ctas = plan.total_blocks < sm_count() ? plan.total_blocks : sm_count();
  plan.chunks = a.k / kUChunkK;
  plan.scale_row_bytes = a.groups * 2;
  const size_t smem = kUPackedBufs * kUPackedBytes + 2 * kUXBytes + 16 * 8 * plan.scale_row_bytes + 48 * sizeof(uint64_t);
  if (smem > 220 * 1024) return XDK_ERR_LIMIT;
  CUtensorMap wmap, smap;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.k / 8), static_cast<cuuint64_t>(a.n)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.k / 2)};
    const cuuint32_t box[2] = {kUChunkK / 8, 32};
    const cuuint64_t sdims[2] = {static_cast<cuuint64_t>(a.groups), static_cast<cuuint64_t>(a.n)};
    const cuuint64_t sstrides[1] = {static_cast<cuuint64_t>(a.groups) * 2};
    const cuuint32_t sbox[2] = {static_cast<cuuint32_t>(a.groups), 32};
    static_assert(kUChunkK / 2 == 128, "the packed box is one 128-byte swizzle span wide");
    if (!encode_tiled_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, a.packed, dims, strides, box, true) ||
        !encode_tiled_2d(&smap, CU_TENSOR_MAP_DATA_TYPE_UINT16, a.scales, sdims, sstrides, sbox, false))
      return XDK_ERR_LAUNCH;
  }
  cudaError_t err = cudaFuncSetAttribute(w4a16_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (err != cudaSuccess) return note_launch(err);
  return launch(w4a16_umma_kernel, dim3(plan.ctas), dim3(kUThreads), smem, stream, 1u, a, plan, wmap, smap);
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
  const int max_ctas = 4 * 148;
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
  // tcgen05 kernel: taken where every SM gets at least two 32-column units (measured at K = 4096, M = 16:
  // 18.6 vs 26.0 us at N = 14336, 32.8 vs 42.4 us at N = 28672, but 16.1 vs 12.5 us at N = 4096, where only one
  // TMEM lane quarter per SM has columns to unpack).  XDK_W4A16_UMMA=1 / =0 forces it on (where eligible) / off.
  static const int umma_env = getenv("XDK_W4A16_UMMA") ? (getenv("XDK_W4A16_UMMA")[0] == '1' ? 1 : 0) : -1;
  const bool umma_ok = fast && m > 8 && k % 256 == 0 && group_size >= 64 && a.groups <= 256 && a.groups % 8 == 0 && aligned16(scales);
  const bool use_umma = umma_env >= 0 ? umma_env == 1 : n >= 64LL * sm_count();
  if (use_umma && umma_ok) {
    const int st = launch_umma(a, s);
    if (st != XDK_ERR_LIMIT) return st;
  }
  if (fast && k % 128 == 0 && m >= 3) return m > 8 ? launch_stream<16>(a, s) : launch_stream<8>(a, s);
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
