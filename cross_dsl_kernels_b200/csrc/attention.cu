// Paged decode attention: one query token per sequence against the K/V cache the append kernel writes.
//
//   out[t][h] = sum_j softmax_j( scale * q[t][h] . K[seq(t)][j][h / G] ) * V[seq(t)][j][h / G],   j = 0 .. positions[t]
//
// (the token's own K/V are in the cache already: the append runs first), G = q_heads / kv_heads query heads
// sharing one KV head.  Pages are found through page_table exactly as the append kernel finds them, in the NHD
// ([page][offset][head][dim]) or HND ([page][head][offset][dim]) cache layout.  Not part of upstream, which stops
// at the append; it is the op that reads what this library's append writes.
//
// HBM-bound: every K and V row of the context is read once (2 * dim * sizeof(T) bytes per position and KV head)
// and used for all G heads of its group.  Work is cut as (context split, KV head, token): a CTA of four warps walks
// its slice of the context in tiles of 32 positions per warp.
//   scores : the warp copies the tile's 32 K rows into shared memory with cp.async, two rows per instruction (a lane
//            reading its own row straight from global memory touches 32 lines per instruction and caps the kernel at
//            a third of the HBM rate); then a lane owns one position: it reads that row from shared memory (row pitch
//            padded by 16 bytes: conflict-free) and accumulates the G dot products against q (FP32 in shared
//            memory, broadcast reads); no shuffles.
//   softmax: per warp and head, running maximum and sum (online softmax) -- one warp max per tile and head.
//   values : lanes turn to own dim/32 dims each; the tile's probabilities and row addresses go through shared
//            memory (one broadcast read per position); the V rows were staged together with the K rows (head sizes
//            whose tiles would leave too few CTAs per SM read them straight from global memory instead).
// 16-bit caches take the tensor-core variant further down: same staging and merges, both contractions as mma tiles.
// The four warps' partial (max, sum, accumulator) are merged in shared memory; the slices of one (token, KV head)
// form a thread-block cluster and are merged in rank order through distributed shared memory, so there is no
// scratch buffer, no second launch, and the result is deterministic.
#include <cooperative_groups.h>
#include <math.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace xdk {
namespace {

constexpr int kAttnWarps = 4;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kMaxSplits = 8;  // portable cluster size
__device__ __forceinline__ int warp_of(unsigned tid) { return static_cast<int>(tid >> 5); }

struct AttnArgs {
  const int64_t* positions;
  const int64_t* page_table;
  const int64_t* sequence_ids;
  int64_t max_pages, page_size;
  int q_heads, kv_heads;
  int hnd;
  float scale;
};

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Merges partial (m, l, acc) `b` into `a` (online softmax): both cover disjoint position sets.
__device__ __forceinline__ void merge_stats(float& m_a, float& l_a, float& scale_a, float& scale_b, float m_b, float l_b) {
  const float m = fmaxf(m_a, m_b);
  scale_a = m_a == -INFINITY ? 0.0f : __expf(m_a - m);
  scale_b = m_b == -INFINITY ? 0.0f : __expf(m_b - m);
  l_a = l_a * scale_a + l_b * scale_b;
  m_a = m;
}

template <typename T, int D>
struct StageV {  // whether a warp's V rows are staged in shared memory beside its K rows
  static constexpr bool value = static_cast<size_t>(kAttnWarps) * 32 * (2 * D * sizeof(T) + 16) <= 72 * 1024;
};

template <typename T, int G, int D>
__global__ void __launch_bounds__(kAttnThreads)
paged_decode_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                              const PeerOut out, AttnArgs a, int splits) {
  constexpr int E = 16 / sizeof(T);   // elements per 16-byte piece
  constexpr int PIECES = D / E;       // pieces per row
  constexpr int DPL = D / 32;         // dims per lane in the value phase
  static_assert(D % 32 == 0 && D % E == 0, "head_dim must be a multiple of 32");
  constexpr int kRowPitch = D * static_cast<int>(sizeof(T)) + 16;  // bytes; the pad spreads the lanes' rows over the banks
  extern __shared__ __align__(16) unsigned char attn_smem[];
  constexpr int kVPitch = D * static_cast<int>(sizeof(T));         // V rows are read along the row: no pad needed
  // V is staged beside K while that leaves room for three CTAs per SM; longer rows read V straight from global memory
  constexpr bool kStageV = StageV<T, D>::value;
  constexpr int kWarpTile = 32 * (kRowPitch + (kStageV ? kVPitch : 0));
  // [warp][32 K rows of kRowPitch | 32 V rows]; reused after the loop for the warps' accumulators [warp][G][D] floats
  unsigned char* ktile = attn_smem + warp_of(threadIdx.x) * kWarpTile;
  unsigned char* vtile = ktile + 32 * kRowPitch;
  float (*part_acc)[G][D] = reinterpret_cast<float (*)[G][D]>(attn_smem);
  __shared__ __align__(16) float qs[G][D];                 // q of the group, pre-multiplied by scale
  __shared__ __align__(16) float probs[kAttnWarps][32][G];  // the tile's probabilities, [position][head]
  __shared__ int64_t rows[kAttnWarps][32];                  // the tile's row offsets (elements)
  __shared__ float part_m[kAttnWarps][G], part_l[kAttnWarps][G];
  __shared__ float cta_m[G], cta_l[G];                      // the CTA's merged (max, sum)

  pdl_launch_dependents();
  pdl_wait();  // q and the caches are the preceding kernels' output
  const int split = blockIdx.x, kvh = blockIdx.y, token = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t ctx = a.positions[token] + 1;
  const int64_t seq = a.sequence_ids[token];
  const int64_t* table = a.page_table + seq * a.max_pages;
  // this CTA's slice of the context: whole tiles of 128 positions, dealt evenly to the splits
  const int64_t tiles = (ctx + kAttnThreads - 1) / kAttnThreads;
  const int64_t t0 = tiles * split / splits, t1 = tiles * (split + 1) / splits;

  for (int i = threadIdx.x; i < G * D; i += kAttnThreads) {
    const int g = i / D, d = i - g * D;
    qs[g][d] = Elem<T>::to_f32(q[(static_cast<int64_t>(token) * a.q_heads + kvh * G + g) * D + d]) * a.scale;
  }
  __syncthreads();

  float m[G], l[G], acc[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY, l[g] = 0.0f;
#pragma unroll
    for (int e = 0; e < DPL; ++e) acc[g][e] = 0.0f;
  }

  for (int64_t tile = t0; tile < t1; ++tile) {
    // ---- scores: this lane's position
    const int64_t j = tile * kAttnThreads + warp * 32 + lane;
    const bool live = j < ctx;
    int64_t row = 0;
    if (live) {
      const int64_t logical = j / a.page_size, off = j - logical * a.page_size;
      const int64_t page = __ldg(table + logical);
      row = a.hnd ? ((page * a.kv_heads + kvh) * a.page_size + off) * D : ((page * a.page_size + off) * a.kv_heads + kvh) * D;
    }
    rows[warp][lane] = row;  // dead positions point at row 0: a valid address, and their probability is 0
    __syncwarp();
    // the tile's K and V rows into shared memory: chunk c = 16-byte piece (c % PIECES) of row (c / PIECES).  Both
    // go out together, so a tile costs one trip to HBM (V read row by row after the scores cost eight more)
#pragma unroll
    for (int i = 0; i < PIECES; ++i) {
      const int c = i * 32 + lane, r = c / PIECES, p = c - r * PIECES;
      cp_async16(ktile + r * kRowPitch + p * 16, reinterpret_cast<const unsigned char*>(k_cache + rows[warp][r]) + p * 16);
    }
    if constexpr (kStageV) {
#pragma unroll
      for (int i = 0; i < PIECES; ++i) {
        const int c = i * 32 + lane, r = c / PIECES, p = c - r * PIECES;
        cp_async16(vtile + r * kVPitch + p * 16, reinterpret_cast<const unsigned char*>(v_cache + rows[warp][r]) + p * 16);
      }
    }
    cp_async_wait_all();
    __syncwarp();
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = 0.0f;
    {
      const unsigned char* mine = ktile + lane * kRowPitch;
#pragma unroll 8
      for (int p = 0; p < PIECES; ++p) {
        const U4 raw = *reinterpret_cast<const U4*>(mine + p * 16);
        const T* kv = reinterpret_cast<const T*>(&raw);
        float kf[E];
#pragma unroll
        for (int e = 0; e < E; ++e) kf[e] = Elem<T>::to_f32(kv[e]);
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
          for (int e = 0; e < E; e += 4) {
            const float4 qv = *reinterpret_cast<const float4*>(&qs[g][p * E + e]);
            s[g] = fmaf(kf[e], qv.x, s[g]);
            s[g] = fmaf(kf[e + 1], qv.y, s[g]);
            s[g] = fmaf(kf[e + 2], qv.z, s[g]);
            s[g] = fmaf(kf[e + 3], qv.w, s[g]);
          }
        }
      }
    }
    // ---- softmax bookkeeping of the tile (per warp)
    float corr[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mx = live ? s[g] : -INFINITY;
#pragma unroll
      for (int sh = 16; sh > 0; sh >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sh));
      const float m_new = fmaxf(m[g], mx);
      corr[g] = m[g] == -INFINITY ? 0.0f : __expf(m[g] - m_new);
      const float p = live ? __expf(s[g] - m_new) : 0.0f;
      l[g] = l[g] * corr[g] + p;  // per-lane share of the sum; lanes are added at the end
      m[g] = m_new;
      probs[warp][lane][g] = p;
    }
    __syncwarp();
    // ---- values: lanes own DPL dims each
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int e = 0; e < DPL; ++e) acc[g][e] *= corr[g];
    const int64_t left = ctx - (tile * kAttnThreads + warp * 32);
    const int n_live = left >= 32 ? 32 : (left > 0 ? static_cast<int>(left) : 0);
    if constexpr (kStageV) {
    for (int j0 = 0; j0 < n_live; ++j0) {
      float vf[DPL];
      const T* vp = reinterpret_cast<const T*>(vtile + j0 * kVPitch) + lane * DPL;
      if constexpr (DPL * sizeof(T) == 8) {
        const uint2 raw = *reinterpret_cast<const uint2*>(vp);
        const T* ve = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int e = 0; e < DPL; ++e) vf[e] = Elem<T>::to_f32(ve[e]);
      } else if constexpr (DPL * sizeof(T) == 16) {
        const U4 raw = *reinterpret_cast<const U4*>(vp);
        const T* ve = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int e = 0; e < DPL; ++e) vf[e] = Elem<T>::to_f32(ve[e]);
      } else {
#pragma unroll
        for (int e = 0; e < DPL; ++e) vf[e] = Elem<T>::to_f32(vp[e]);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float p = probs[warp][j0][g];
#pragma unroll
        for (int e = 0; e < DPL; ++e) acc[g][e] = fmaf(p, vf[e], acc[g][e]);
      }
    }
    } else {
    // four positions per pass, their V loads issued together (dead positions carry probability 0 and row 0)
    for (int j0 = 0; j0 < n_live; j0 += 4) {
      float vf[4][DPL];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const T* vp = v_cache + rows[warp][j0 + u] + lane * DPL;
        if constexpr (DPL * sizeof(T) == 8) {
          const uint2 raw = __ldg(reinterpret_cast<const uint2*>(vp));
          const T* ve = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int e = 0; e < DPL; ++e) vf[u][e] = Elem<T>::to_f32(ve[e]);
        } else if constexpr (DPL * sizeof(T) == 16) {
          const U4 raw = ld_stream16(vp);
          const T* ve = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int e = 0; e < DPL; ++e) vf[u][e] = Elem<T>::to_f32(ve[e]);
        } else {
#pragma unroll
          for (int e = 0; e < DPL; ++e) vf[u][e] = Elem<T>::to_f32(vp[e]);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float p = probs[warp][j0 + u][g];
#pragma unroll
          for (int e = 0; e < DPL; ++e) acc[g][e] = fmaf(p, vf[u][e], acc[g][e]);
        }
    }
    }
    __syncwarp();  // the tile's shared entries are free for the next tile
  }

  // ---- warp totals, then the four warps of the CTA (fixed order)
  __syncthreads();  // every warp is done with its K tile: the buffer now holds the accumulators
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float sum = l[g];  // every lane scaled its share by the same corrections, so shares can simply be added
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, sh);
    if (lane == 0) part_m[warp][g] = m[g], part_l[warp][g] = sum;
#pragma unroll
    for (int e = 0; e < DPL; ++e) part_acc[warp][g][lane * DPL + e] = acc[g][e];
  }
  __syncthreads();
  // thread (g, d) pairs merge the warps; results land in slot 0
  for (int i = threadIdx.x; i < G * D; i += kAttnThreads) {
    const int g = i / D, d = i - g * D;
    float mm = part_m[0][g], ll = part_l[0][g], aa = part_acc[0][g][d];
    for (int w = 1; w < kAttnWarps; ++w) {
      float sa, sb;
      merge_stats(mm, ll, sa, sb, part_m[w][g], part_l[w][g]);
      aa = aa * sa + part_acc[w][g][d] * sb;
    }
    part_acc[0][g][d] = aa;
    if (d == 0) cta_m[g] = mm, cta_l[g] = ll;
  }
  __syncthreads();

  if (splits > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();  // every slice's partial is in its CTA's shared memory
    if (split == 0) {
      for (int i = threadIdx.x; i < G * D; i += kAttnThreads) {
        const int g = i / D, d = i - g * D;
        float mm = cta_m[g], ll = cta_l[g], aa = part_acc[0][g][d];
        for (int r = 1; r < splits; ++r) {  // rank order
          const float mr = *cluster.map_shared_rank(&cta_m[g], r), lr = *cluster.map_shared_rank(&cta_l[g], r);
          const float ar = *cluster.map_shared_rank(&part_acc[0][g][d], r);
          float sa, sb;
          merge_stats(mm, ll, sa, sb, mr, lr);
          aa = aa * sa + ar * sb;
        }
        peer_store(out, token, (kvh * G + g) * D + d, Elem<T>::from_f32(aa / ll));
      }
    }
    cluster.sync();  // nobody leaves while rank 0 may still read its shared memory
  } else {
    for (int i = threadIdx.x; i < G * D; i += kAttnThreads) {
      const int g = i / D, d = i - g * D;
      peer_store(out, token, (kvh * G + g) * D + d, Elem<T>::from_f32(part_acc[0][g][d] / cta_l[g]));
    }
  }
}

// ---- the same kernel with both contractions on the tensor cores (16-bit caches) --------------------------------
// The lane-per-position kernel above spends ~1700 warp instructions per tile of 32 positions (two FMAs per cache
// element and G heads) and is issue-bound at ~0.6 of the HBM rate.  Here the G query heads of the group are the
// (zero-padded) 16 rows of mma.m16n8k16 tiles: S = Q K^T with K rows as the "col" operand straight from the staged
// tile (ldmatrix), P V with V through ldmatrix.trans, P rounded to the cache type, FP32 accumulators in registers.
// Everything else (staging, online softmax per head, merges) is as above.
template <typename T> struct Mma16816;
template <> struct Mma16816<__half> {
  // rows 8-15 of A are zero, so rows 8-15 of the result are not kept: two accumulator registers per tile, not four
  __device__ static __forceinline__ void run(float (&d)[2], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    float unused2, unused3;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%10};"
                 : "+f"(d[0]), "+f"(d[1]), "=f"(unused2), "=f"(unused3)
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.0f));
  }
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};
template <> struct Mma16816<__nv_bfloat16> {
  __device__ static __forceinline__ void run(float (&d)[2], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    float unused2, unused3;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%10};"
                 : "+f"(d[0]), "+f"(d[1]), "=f"(unused2), "=f"(unused3)
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.0f));
  }
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem_row)));
}

template <typename T, int G, int D>
__global__ void __launch_bounds__(kAttnThreads, D <= 128 ? 3 : 1)
paged_decode_attention_tc_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                 const PeerOut out, AttnArgs a, int splits) {
  static_assert(sizeof(T) == 2 && G <= 8 && D % 32 == 0, "16-bit caches, at most eight heads per group");
  constexpr int PIECES = D / 8;                 // 16-byte pieces per row
  constexpr int kPitch = D * 2 + 16;            // bytes; the pad keeps the eight rows of an ldmatrix on eight bank groups
  constexpr int kWarpTile = 2 * 32 * kPitch;    // K rows, then V rows
  extern __shared__ __align__(16) unsigned char attn_smem[];
  unsigned char* ktile = attn_smem + warp_of(threadIdx.x) * kWarpTile;
  unsigned char* vtile = ktile + 32 * kPitch;
  float (*part_acc)[G][D] = reinterpret_cast<float (*)[G][D]>(attn_smem);
  __shared__ int64_t rows[kAttnWarps][32];
  __shared__ float part_m[kAttnWarps][G], part_l[kAttnWarps][G];
  __shared__ float cta_m[G], cta_l[G];

  pdl_launch_dependents();
  pdl_wait();  // q and the caches are the preceding kernels' output
  const int split = blockIdx.x, kvh = blockIdx.y, token = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grow = lane >> 2, quad = lane & 3;  // fragment row (= head of the group when < G), position inside the quad
  const bool head_live = grow < G;
  const int64_t ctx = a.positions[token] + 1;
  const int64_t seq = a.sequence_ids[token];
  const int64_t* table = a.page_table + seq * a.max_pages;
  const int64_t tiles = (ctx + kAttnThreads - 1) / kAttnThreads;
  const int64_t t0 = tiles * split / splits, t1 = tiles * (split + 1) / splits;

  // Q as A fragments: a0 = (row grow, dims 16 ks + 2 quad + {0,1}), a2 = the same + 8 dims; rows >= G are zero
  uint32_t qa0[D / 16], qa2[D / 16];
  {
    const T* qrow = q + (static_cast<int64_t>(token) * a.q_heads + kvh * G + (head_live ? grow : 0)) * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qa0[ks] = head_live ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + quad * 2) : 0u;
      qa2[ks] = head_live ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + quad * 2 + 8) : 0u;
    }
  }
  float m_run = -INFINITY, l_run = 0.0f;  // of head grow; l_run is this thread's share of the sum
  float o[D / 8][2];
#pragma unroll
  for (int nd = 0; nd < D / 8; ++nd) o[nd][0] = o[nd][1] = 0.0f;

  for (int64_t tile = t0; tile < t1; ++tile) {
    const int64_t base = tile * kAttnThreads + warp * 32;
    {
      const int64_t j = base + lane;
      int64_t row = 0;
      if (j < ctx) {
        const int64_t logical = j / a.page_size, off = j - logical * a.page_size;
        const int64_t page = __ldg(table + logical);
        row = a.hnd ? ((page * a.kv_heads + kvh) * a.page_size + off) * D : ((page * a.page_size + off) * a.kv_heads + kvh) * D;
      }
      rows[warp][lane] = row;  // dead positions point at row 0: a valid address, and their probability is 0
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < PIECES; ++i) {
      const int c = i * 32 + lane, r = c / PIECES, p = c - r * PIECES;
      cp_async16(ktile + r * kPitch + p * 16, reinterpret_cast<const unsigned char*>(k_cache + rows[warp][r]) + p * 16);
    }
#pragma unroll
    for (int i = 0; i < PIECES; ++i) {
      const int c = i * 32 + lane, r = c / PIECES, p = c - r * PIECES;
      cp_async16(vtile + r * kPitch + p * 16, reinterpret_cast<const unsigned char*>(v_cache + rows[warp][r]) + p * 16);
    }
    cp_async_wait_all();
    __syncwarp();

    // ---- S = Q K^T: four n-tiles of eight positions; lane supplies the address of row (lane % 8) of matrix lane / 8
    float sc[4][2];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      sc[nt][0] = sc[nt][1] = 0.0f;
      const unsigned char* krow = ktile + (nt * 8 + (lane & 7)) * kPitch + (lane >> 3) * 16;
#pragma unroll
      for (int ks = 0; ks < D / 16; ks += 2) {  // one ldmatrix.x4 = the (b0, b1) of two k slices
        uint32_t b[4];
        ldmatrix_x4(b, krow + ks * 32);
        Mma16816<T>::run(sc[nt], qa0[ks], qa2[ks], b[0], b[1]);
        Mma16816<T>::run(sc[nt], qa0[ks + 1], qa2[ks + 1], b[2], b[3]);
      }
    }
    // ---- online softmax of head grow: this thread holds positions base + 8 nt + 2 quad + {0, 1}
    float mx = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const bool live = base + nt * 8 + quad * 2 + e < ctx;
        sc[nt][e] = live ? sc[nt][e] * a.scale : -INFINITY;
        mx = fmaxf(mx, sc[nt][e]);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float corr = m_run == -INFINITY ? 0.0f : __expf(m_run - m_new);
    uint32_t pa[4];  // P as A fragments: k slice kp = positions 16 kp .. 16 kp + 15: a0 from n-tile 2 kp, a2 from 2 kp + 1
    float psum = 0.0f;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const float p0 = sc[nt][0] == -INFINITY ? 0.0f : __expf(sc[nt][0] - m_new);
      const float p1 = sc[nt][1] == -INFINITY ? 0.0f : __expf(sc[nt][1] - m_new);
      psum += p0 + p1;
      pa[nt] = Mma16816<T>::pack(p0, p1);
    }
    l_run = l_run * corr + psum;
    m_run = m_new;
#pragma unroll
    for (int nd = 0; nd < D / 8; ++nd) o[nd][0] *= corr, o[nd][1] *= corr;
    // ---- O += P V: V^T through ldmatrix.trans; matrix lane / 8 = (position half, dim tile)
#pragma unroll
    for (int kp = 0; kp < 2; ++kp) {
      const unsigned char* vrow = vtile + (kp * 16 + (lane >> 3 & 1) * 8 + (lane & 7)) * kPitch + (lane >> 4) * 16;
#pragma unroll
      for (int nd = 0; nd < D / 8; nd += 2) {  // one ldmatrix.x4.trans = the (b0, b1) of two dim tiles
        uint32_t b[4];
        ldmatrix_x4_trans(b, vrow + nd * 16);
        Mma16816<T>::run(o[nd], pa[2 * kp], pa[2 * kp + 1], b[0], b[1]);
        Mma16816<T>::run(o[nd + 1], pa[2 * kp], pa[2 * kp + 1], b[2], b[3]);
      }
    }
    __syncwarp();  // the tile's shared entries are free for the next tile
  }

  // ---- warp totals, then the four warps of the CTA (fixed order)
  __syncthreads();  // every warp is done with its tiles: the buffer now holds the accumulators
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if (head_live) {
    if (quad == 0) part_m[warp][grow] = m_run, part_l[warp][grow] = l_run;
#pragma unroll
    for (int nd = 0; nd < D / 8; ++nd) {
      part_acc[warp][grow][nd * 8 + quad * 2] = o[nd][0];
      part_acc[warp][grow][nd * 8 + quad * 2 + 1] = o[nd][1];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += kAttnThreads) {
    const int g = i / D, d = i - g * D;
    float mm = part_m[0][g], ll = part_l[0][g], aa = part_acc[0][g][d];
    for (int w = 1; w < kAttnWarps; ++w) {
      float sa, sb;
      merge_stats(mm, ll, sa, sb, part_m[w][g], part_l[w][g]);
      aa = aa * sa + part_acc[w][g][d] * sb;
    }
    part_acc[0][g][d] = aa;
    if (d == 0) cta_m[g] = mm, cta_l[g] = ll;
  }
  __syncthreads();

  if (splits > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();  // every slice's partial is in its CTA's shared memory
    if (split == 0) {
      for (int i = threadIdx.x; i < G * D; i += kAttnThreads) {
        const int g = i / D, d = i - g * D;
        float mm = cta_m[g], ll = cta_l[g], aa = part_acc[0][g][d];
        for (int r = 1; r < splits; ++r) {  // rank order
          const float mr = *cluster.map_shared_rank(&cta_m[g], r), lr = *cluster.map_shared_rank(&cta_l[g], r);
          const float ar = *cluster.map_shared_rank(&part_acc[0][g][d], r);
          float sa, sb;
          merge_stats(mm, ll, sa, sb, mr, lr);
          aa = aa * sa + ar * sb;
        }
        peer_store(out, token, (kvh * G + g) * D + d, Elem<T>::from_f32(aa / ll));
      }
    }
    cluster.sync();  // nobody leaves while rank 0 may still read its shared memory
  } else {
    for (int i = threadIdx.x; i < G * D; i += kAttnThreads) {
      const int g = i / D, d = i - g * D;
      peer_store(out, token, (kvh * G + g) * D + d, Elem<T>::from_f32(part_acc[0][g][d] / cta_l[g]));
    }
  }
}

// launch_opts puts the cluster along y; this kernel's cluster runs along x (the context splits)
template <typename T, int G, int D>
int launch_attention_cluster(const void* q, const void* kc, const void* vc, const PeerOut& out, const AttnArgs& a, int64_t tokens,
                             int splits, cudaStream_t s) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(splits), static_cast<unsigned>(a.kv_heads), static_cast<unsigned>(tokens));
  cfg.blockDim = dim3(kAttnThreads);
  constexpr bool kTensorCores = sizeof(T) == 2;  // 16-bit caches: both contractions as mma.sync tiles
  constexpr size_t tile_bytes = kTensorCores ? static_cast<size_t>(kAttnWarps) * 2 * 32 * (D * sizeof(T) + 16)
                                             : static_cast<size_t>(kAttnWarps) * 32 * ((StageV<T, D>::value ? 2 : 1) * D * sizeof(T) + 16);
  constexpr size_t acc_bytes = static_cast<size_t>(kAttnWarps) * G * D * sizeof(float);
  constexpr size_t smem = tile_bytes > acc_bytes ? tile_bytes : acc_bytes;
  void (*kernel)(const T*, const T*, const T*, const PeerOut, AttnArgs, int);
  if constexpr (kTensorCores) kernel = paged_decode_attention_tc_kernel<T, G, D>;
  else kernel = paged_decode_attention_kernel<T, G, D>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) return note_launch(err);
  }
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (splits > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = static_cast<unsigned>(splits);
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (call_flags() & XDK_DEPENDENT_LAUNCH) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return note_launch(cudaLaunchKernelEx(&cfg, kernel, static_cast<const T*>(q), static_cast<const T*>(kc),
                                        static_cast<const T*>(vc), out, a, splits));
}

template <typename T, int G>
int dispatch_dim(int64_t d, const void* q, const void* kc, const void* vc, const PeerOut& out, const AttnArgs& a, int64_t tokens, int splits,
                 cudaStream_t s) {
  switch (d) {
    case 64: return launch_attention_cluster<T, G, 64>(q, kc, vc, out, a, tokens, splits, s);
    case 128: return launch_attention_cluster<T, G, 128>(q, kc, vc, out, a, tokens, splits, s);
    case 256: return launch_attention_cluster<T, G, 256>(q, kc, vc, out, a, tokens, splits, s);
    default: return XDK_ERR_LIMIT;
  }
}

template <typename T>
int dispatch_group(int g, int64_t d, const void* q, const void* kc, const void* vc, const PeerOut& out, const AttnArgs& a, int64_t tokens,
                   int splits, cudaStream_t s) {
  switch (g) {
    case 1: return dispatch_dim<T, 1>(d, q, kc, vc, out, a, tokens, splits, s);
    case 2: return dispatch_dim<T, 2>(d, q, kc, vc, out, a, tokens, splits, s);
    case 4: return dispatch_dim<T, 4>(d, q, kc, vc, out, a, tokens, splits, s);
    case 8: return dispatch_dim<T, 8>(d, q, kc, vc, out, a, tokens, splits, s);
    default: return XDK_ERR_LIMIT;
  }
}

}  // namespace
}  // namespace xdk

extern "C" int xdk_paged_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int64_t* positions,
                                          const int64_t* page_table, const int64_t* sequence_ids, void* out, int64_t tokens,
                                          int64_t q_heads, int64_t kv_heads, int64_t head_dim, int64_t max_pages_per_seq,
                                          int64_t page_size, int cache_is_hnd, float scale, int64_t context_hint, int dtype,
                                          unsigned flags, void* stream) {
  if (!out) return XDK_ERR_ARG;
  xdk_peer_out one = {};
  one.ptr[0] = out, one.world = 1, one.ld = q_heads * head_dim, one.col0 = 0;
  return xdk_paged_decode_attention_peer(q, k_cache, v_cache, positions, page_table, sequence_ids, &one, tokens, q_heads, kv_heads,
                                         head_dim, max_pages_per_seq, page_size, cache_is_hnd, scale, context_hint, dtype, flags,
                                         stream);
}

extern "C" int xdk_paged_decode_attention_peer(const void* q, const void* k_cache, const void* v_cache, const int64_t* positions,
                                               const int64_t* page_table, const int64_t* sequence_ids, const xdk_peer_out* out_dst,
                                               int64_t tokens, int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                                               int64_t max_pages_per_seq, int64_t page_size, int cache_is_hnd, float scale,
                                               int64_t context_hint, int dtype, unsigned flags, void* stream) {
  using namespace xdk;
  PeerOut out;
  if (int st = make_out(out_dst, nullptr, 1, &out)) return st;
  if (q_heads > 0 && head_dim > 0 && out.ld < out.col0 + q_heads * head_dim) return XDK_ERR_ARG;
  if (flags & ~XDK_DEPENDENT_LAUNCH) return XDK_ERR_ARG;
  CallFlagsScope scope(flags);
  if (!q || !k_cache || !v_cache || !positions || !page_table || !sequence_ids) return XDK_ERR_ARG;
  if (tokens < 1 || q_heads < 1 || kv_heads < 1 || head_dim < 1 || max_pages_per_seq < 1 || page_size < 1) return XDK_ERR_ARG;
  if (q_heads % kv_heads != 0 || !(scale == scale)) return XDK_ERR_ARG;
  if (tokens > 65535 || kv_heads > 65535) return XDK_ERR_LIMIT;
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache)) return XDK_ERR_ARG;
  if (int st = require_sm100()) return st;
  AttnArgs a;
  a.positions = positions, a.page_table = page_table, a.sequence_ids = sequence_ids;
  a.max_pages = max_pages_per_seq, a.page_size = page_size;
  a.q_heads = static_cast<int>(q_heads), a.kv_heads = static_cast<int>(kv_heads);
  a.hnd = cache_is_hnd ? 1 : 0;
  a.scale = scale;
  // Context splits: as many CTAs as the SMs hold at once, at most one split per 128-position tile of the longest
  // context the caller expects (context_hint; <= 0: assume long contexts), at most the portable cluster size.
  // CTAs an SM holds at once, by the shared memory of the kernel that will run (registers allow four)
  const int64_t elem = dtype == XDK_F32 ? 4 : 2;
  const bool staged = kAttnWarps * 32 * (2 * head_dim * elem + 16) <= 72 * 1024;  // StageV of the FP32 kernel
  const int64_t tile_smem = dtype == XDK_F32 ? kAttnWarps * 32 * ((staged ? 2 : 1) * head_dim * elem + 16)
                                            : kAttnWarps * 2 * 32 * (head_dim * elem + 16);
  int64_t resident = (220 * 1024) / (tile_smem > 0 ? tile_smem : 1);
  resident = resident < 1 ? 1 : (resident > 4 ? 4 : resident);
  int splits = static_cast<int>(resident * sm_count() / (tokens * kv_heads));      // one wave, never a partial second one
  if (context_hint > 0) {
    const int64_t tiles = (context_hint + kAttnThreads - 1) / kAttnThreads;
    if (splits > tiles) splits = static_cast<int>(tiles);
  }
  if (splits > kMaxSplits) splits = kMaxSplits;
  if (splits < 1) splits = 1;
  const int g = static_cast<int>(q_heads / kv_heads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case XDK_F32: return dispatch_group<float>(g, head_dim, q, k_cache, v_cache, out, a, tokens, splits, s);
    case XDK_BF16: return dispatch_group<__nv_bfloat16>(g, head_dim, q, k_cache, v_cache, out, a, tokens, splits, s);
    case XDK_F16: return dispatch_group<__half>(g, head_dim, q, k_cache, v_cache, out, a, tokens, splits, s);
    default: return XDK_ERR_ARG;
  }
}
