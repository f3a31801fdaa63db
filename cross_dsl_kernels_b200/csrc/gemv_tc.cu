// FP32 small-M projection on the 5th-generation tensor cores (tcgen05, kind::tf32) with FP32-grade accuracy.
//
// y[M, N] = x[M, K] . W + bias for 4 < M <= 16.  On CUDA cores this shape is bound by FP32 operand delivery
// (16 rows of x against every weight), not by HBM; the tensor cores have the throughput, but a TF32 product keeps
// only 11 significant bits of each operand.  So every operand is split into two TF32 numbers,
//     v = hi + lo,   hi = v with the low 13 mantissa bits cleared,   lo = v - hi  (exact in FP32),
// and the product is formed as hi.hi + hi.lo + lo.hi -- three MMAs per k block, FP32 accumulation in TMEM.  The
// dropped lo.lo term and the bits of lo the tensor core ignores are below 2^-21 relative per product.  The
// accumulation inside the tensor core may truncate instead of rounding; to keep that bias small the sum is spread
// over up to sixteen accumulators per k range that are added in FP32 in a fixed order at the end, so results are
// deterministic.  Measured against an FP64 product the relative L2 error is ~1e-6, inside the 1e-5 gate of the
// projection; callers that need strict FP32 FMA arithmetic pass scratch to xdk_gemv_f32 and get the CUDA-core
// tile-stream kernel instead.
//
// Layout of the work (same scheme as the W4A16 tcgen05 kernel): operands are swapped so that the UMMA "M"
// dimension (128 TMEM lanes) carries output columns, D[128 lanes x 16 S] += A[128 x 8 k] * B[8 k x 16 S], A = W (split)
// in tensor memory, B = x^T (split) in shared memory.  One persistent CTA per SM owns an evenly dealt range of
// 32-column units and walks it in strips of <= 4 units, full K each; narrow strips split K S ways over the TMEM
// lane quarters and add the S partial sums through shared memory in a fixed order; S is one value per launch
// (4 when no CTA has more than one unit, 2 for two, else 1), which also sizes the x buffers, and whatever shared
// memory they leave goes to the W ring.  A projection with fewer units than half the SMs (a column shard of a
// multi-GPU run) is additionally split along K over the 2 or 4 CTAs of a thread-block cluster: every CTA of the
// cluster walks the same strips over its own part of K, the parts store their partial sums into the rank-0 CTA's
// shared memory (distributed shared memory, mbarrier hand-off with bounded waits) and rank 0 adds them in rank
// order, so the result stays deterministic.
//   TMA warps (4)      : one lane each, one warp per TMEM lane quarter: the W tile of a 64-k step (NK: two 128-byte
//                        swizzled [32 columns][32 k] boxes per quarter; KN: one [64 k][32 u columns] box per k range,
//                        u = units of the strip, so that HBM sees runs of up to 512 bytes) into a ring of step buffers.  Four warps because a warp gets a TMA box copy out only every ~230
//                        cycles: one producer issuing all boxes of a step was the bottleneck (NK slower than KN)
//   x warps (2)        : one lane issues one TMA box per k range ([16 rows][64 k]); both warps split every 16-byte
//                        unit into hi and lo and move it to its place in the two K-major core-matrix operand images
//   split warps (8)    : thread = one TMEM lane = one output column; warp w owns lane quarter w % 4 and k half
//                        w / 4 of every step: shared loads -> hi/lo -> tcgen05.st into the stage's hi and lo columns
//   MMA warps (4)      : one lane each.  A warp gets a tcgen05.mma out only every ~118 cycles whatever the shape,
//                        but warps issue side by side (measured: 8 warps, one MMA per 15 cycles in aggregate), so
//                        the 8 k blocks of a step are dealt round-robin to 4 issuers (3 MMAs per block), each with
//                        its own accumulators
//   split warps 0-3    : epilogue -- tcgen05.ld of the accumulators, fixed-order sum, bias, FP32 store
// TMEM columns (512): (256 / issuers) i + 16 S a .. accumulator a of issuer i, 256 + 128 s .. stage s (64 hi columns, 64 lo).
// Every wait is time-bounded; on a timeout the kernel raises a fault word, stops issuing work, and still frees
// its TMEM columns before it returns.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "common.cuh"
#include "umma.cuh"

namespace xdk {
namespace {

__device__ unsigned int g_tc_fault;  // set when a bounded wait gives up

constexpr int kStepK = 64;                      // k per step
constexpr int kMaxK = 16384;                    // largest K the split-TF32 accumulation keeps inside the 1e-5 gate
constexpr int kMaxRing = 8;                     // W step buffers: as many as shared memory leaves (plan.ring)
constexpr int kQuarterBytes = 32 * kStepK * 4;  // one lane quarter's tile: 32 columns x 64 k
constexpr int kStepBytes = 4 * kQuarterBytes;
constexpr int kStages = 2;                      // A stages in TMEM
constexpr int kStageCols = 2 * kStepK;          // hi columns then lo columns
constexpr int kMaxIssuers = 4;
constexpr int kAccRegion = 256;                 // TMEM columns for accumulators: 256 / issuers each, 16 S per accumulator
constexpr int kTmemCols = 512;
constexpr int kTmemA = kAccRegion;
static_assert(kTmemA + kStages * kStageCols <= kTmemCols, "stages must fit the TMEM allocation");
constexpr int kXLbo = 128, kXSbo = (kStepK / 4) * kXLbo;  // x image: [row group of 8][16 k groups][8 rows x 16 B]
constexpr int kXHalf1 = 2 * kXSbo;              // hi (or lo) image of one k range: 16 rows
constexpr int kXRaw1 = 16 * kStepK * 4;         // one k range of [16 rows][64 k] as TMA lands it
constexpr int kXBufs = 2;
constexpr int kRedBytes = 128 * 16 * 4;         // k-range partials: [lane][16] floats
constexpr int kMaxParts = 4;                    // CTAs of a cluster sharing a strip along K
constexpr int kWTma = 8, kWX0 = 12, kWMma0 = 14;  // warp roles; 0-7 split, 8-11 TMA, 12-13 x, 14-17 MMA
constexpr int kThreads = (kWMma0 + kMaxIssuers) * 32;
constexpr uint32_t kHiMask = 0xffffe000u;       // keeps sign, exponent and the 10 mantissa bits TF32 uses

struct TcArgs {
  const float* bias;
  PeerOut out;
  int m, k, n;
  int ctas, total_units;
  int split;  // k ranges per strip (1, 2, 4), the same for every strip of the launch
  int ring;   // W step buffers
  int kparts; // CTAs of a cluster that share every strip, each walking K / kparts (1, 2, 4); grid = (ctas, kparts)
};

__device__ __forceinline__ void split_tf32(uint32_t v, uint32_t& hi, uint32_t& lo) {
  hi = v & kHiMask;
  lo = __float_as_uint(__fsub_rn(__uint_as_float(v), __uint_as_float(hi)));
}

template <bool NK>
__global__ void __launch_bounds__(kThreads, 1)
gemv_tc_kernel(TcArgs a, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap wmap2,
               const __grid_constant__ CUtensorMap wmap3, const __grid_constant__ CUtensorMap wmap4,
               const __grid_constant__ CUtensorMap xmap) {  // wmap2-4 (KN only): boxes 64, 96, 128 columns wide
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int S = a.split, kRing = a.ring;
  const int issuers = kMaxIssuers, acc_cols = kAccRegion / issuers;
  const int kXHalfBytes = S * kXHalf1, kXBytes = 2 * kXHalfBytes, kXRawBytes = S * kXRaw1;
  unsigned char* ring = smem_raw;                            // [ring][kStepBytes]
  unsigned char* xbuf = ring + kRing * kStepBytes;           // [kXBufs][hi image | lo image], 16 S rows each
  unsigned char* xraw = xbuf + kXBufs * kXBytes;             // [kXBufs][16 rows][S k ranges][64 k]
  float* red = reinterpret_cast<float*>(xraw + kXBufs * kXRawBytes);
  // partial sums of the other CTAs of the cluster land here (in the rank-0 CTA): [part - 1][lane][16] floats
  float* inbox = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(red) + kRedBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(inbox) + (a.kparts - 1) * kRedBytes);
  uint64_t* w_full = bars;                 // [kMaxRing] TMA bytes of a W step landed
  uint64_t* w_empty = w_full + kMaxRing;   // [kMaxRing] the 8 split warps are done with the step
  uint64_t* a_full = w_empty + kMaxRing;   // [kStages] the 8 split warps wrote the stage to TMEM
  uint64_t* a_empty = a_full + kStages;    // [kStages] every issuer's MMAs that read the stage completed
  uint64_t* x_raw = a_empty + kStages;     // [kXBufs]  TMA bytes of an x step landed
  uint64_t* x_full = x_raw + kXBufs;       // [kXBufs]  the x warps wrote both operand images
  uint64_t* x_empty = x_full + kXBufs;     // [kXBufs]  every issuer's MMAs that read the images completed
  uint64_t* acc_full = x_empty + kXBufs;   // [1]
  uint64_t* inbox_full = acc_full + 1;     // [1] rank 0: the other parts stored a strip's partials (128 arrivals each)
  uint64_t* inbox_free = inbox_full + 1;   // [1] other ranks: rank 0 has read the partials of the previous strip
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(inbox_free + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // K split across the CTAs of a cluster (narrow projections: fewer 32-column units than SMs): part p walks
  // k in [p K / kparts, (p + 1) K / kparts) of the SAME strips; rank 0 adds the parts in rank order and stores.
  const int part = a.kparts > 1 ? static_cast<int>(blockIdx.y) : 0;
  const int k_len = a.k / a.kparts, k_base = part * k_len;
  UmmaCursor cur;
  cur.init(blockIdx.x, a.ctas, a.total_units, k_len, kStepK, S);

  if (threadIdx.x == 0) {
    for (int i = 0; i < kRing; ++i) {
      mbar_init(w_full + i, 4);   // one arrival (with its bytes) per TMA warp
      mbar_init(w_empty + i, 8);
    }
    for (int i = 0; i < kXBufs; ++i) {
      mbar_init(x_raw + i, 1);
      mbar_init(x_full + i, 1);
      mbar_init(x_empty + i, issuers);
    }
    for (int i = 0; i < kStages; ++i) {
      mbar_init(a_full + i, 8);
      mbar_init(a_empty + i, issuers);
    }
    mbar_init(acc_full, issuers);
    mbar_init(inbox_full, 128 * (a.kparts - 1) > 0 ? 128 * (a.kparts - 1) : 1);
    mbar_init(inbox_free, 1);
    mbar_fence_init();
  }
  if (warp == kWTma) tmem_alloc<kTmemCols>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  if (a.kparts > 1) {  // every CTA's barriers exist before a peer may arrive on them
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= kWTma && warp < kWX0) {
    // ------------------------------------------------------------ TMA producers: W tiles, one lane quarter each
    if (lane == 0) {
      const int lq = warp - kWTma;
      bool ok = true;
      while (ok && cur.begin_strip()) {
        const int qpk = 4 / cur.split;  // lane quarters per k range = units the strip can hold
        const bool live = lq % qpk < cur.units;
        const int col0 = (cur.unit + lq % qpk) * 32, k_range0 = (lq / qpk) * cur.kper;
        do {
          const int buf = cur.q % kRing;
          if (cur.q >= kRing && !mbar_wait(w_empty + buf, ((cur.q / kRing) - 1) & 1)) {
            ok = false;
            break;
          }
          const int k0 = k_base + k_range0 + cur.kc * kStepK;
          if (NK) {  // two [32 columns][32 k] boxes, 128-byte rows, swizzled
            if (!live) {
              mbar_arrive_cta(w_full + buf);
              continue;
            }
            mbar_expect_tx(w_full + buf, static_cast<unsigned>(kQuarterBytes));
            unsigned char* dst = ring + buf * kStepBytes + lq * kQuarterBytes;
            tma_box_2d(dst, &wmap, k0, col0, w_full + buf);
            tma_box_2d(dst + kQuarterBytes / 2, &wmap, k0 + 32, col0, w_full + buf);
          } else {   // the first quarter of each k range fetches [64 k][32 u columns] for all its quarters
            if (lq % qpk != 0) {
              mbar_arrive_cta(w_full + buf);
              continue;
            }
            mbar_expect_tx(w_full + buf, static_cast<unsigned>(cur.units * kQuarterBytes));
            unsigned char* dst = ring + buf * kStepBytes + lq * kQuarterBytes;
            const CUtensorMap* map = cur.units == 1 ? &wmap : (cur.units == 2 ? &wmap2 : (cur.units == 3 ? &wmap3 : &wmap4));
            tma_box_2d(dst, map, col0, k0, w_full + buf);
          }
        } while (cur.next_step());
      }
      if (!ok) atomicOr(&g_tc_fault, 1u);
    }
  } else if (warp >= kWMma0) {
    // ------------------------------------------------------------ MMA issuers
    if (lane == 0 && warp - kWMma0 < issuers) {
      const int issuer = warp - kWMma0;
      const uint64_t xd0 = umma_desc(smem_u32(xbuf), kXLbo, kXSbo);
      const uint32_t xd_lo = static_cast<uint32_t>(xd0), xd_hi = static_cast<uint32_t>(xd0 >> 32);
      bool ok = true;
      while (ok && cur.begin_strip()) {
        const uint32_t idesc = umma_idesc(16 * cur.split, 2u);
        const int naccs = min(acc_cols / (16 * S), cur.steps);
        do {
          const int xb = cur.q % kXBufs, s = cur.q % kStages;
          ok = mbar_wait(x_full + xb, (cur.q / kXBufs) & 1) && mbar_wait(a_full + s, (cur.q / kStages) & 1);
          if (!ok) break;
          tc_fence_after();
          const int sel = cur.kc % naccs;
          const uint32_t acc = tmem_base + issuer * acc_cols + sel * 16 * S;
          const bool fresh = cur.kc < naccs;  // first step that touches this accumulator in the strip
          const uint32_t a_hi = tmem_base + kTmemA + s * kStageCols + issuer * 8;
          const uint32_t x_lo = xd_lo + ((xb * kXBytes + issuer * 2 * kXLbo) >> 4);
          for (int j = 0; j * issuers < kStepK / 8; ++j) {  // k blocks issuer, issuer + issuers
            uint64_t b_hi, b_lo;
            const uint32_t off = (j * issuers * 2 * kXLbo) >> 4;
            asm("mov.b64 %0, {%1, %2};" : "=l"(b_hi) : "r"(x_lo + off), "r"(xd_hi));
            asm("mov.b64 %0, {%1, %2};" : "=l"(b_lo) : "r"(x_lo + off + (kXHalfBytes >> 4)), "r"(xd_hi));
            const uint32_t ah = a_hi + j * issuers * 8;
            umma_tf32_ta(acc, ah, b_hi, idesc, !(fresh && j == 0));
            umma_tf32_ta(acc, ah, b_lo, idesc, true);
            umma_tf32_ta(acc, ah + kStepK, b_hi, idesc, true);
          }
          umma_commit(a_empty + s);
          umma_commit(x_empty + xb);
        } while (cur.next_step());
        if (ok) umma_commit(acc_full);
      }
      if (!ok) atomicOr(&g_tc_fault, 2u);
    }
  } else if (warp >= kWX0) {  // the two warps between the TMA warps and the MMA warps
    // ------------------------------------------------------------ x warps
    const int t = threadIdx.x - kWX0 * 32;  // 0 .. 63
    bool ok = true;
    UmmaCursor ahead = cur;  // issues the loads, kXBufs steps in front of `cur`
    bool ahead_live = ahead.begin_strip();
    auto issue = [&]() {  // raw buffer ahead.q % kXBufs is free: its last readers passed the x-warp barrier
      if (!ahead_live) return;
      if (t == 0) {
        const int xb = ahead.q % kXBufs;
        mbar_expect_tx(x_raw + xb, static_cast<unsigned>(kXRawBytes));  // rows >= M are out of range: zero-filled, still counted
        tma_box_4d(xraw + xb * kXRawBytes, &xmap, ahead.kc * kStepK, 0, part, 0, x_raw + xb);  // all k ranges in one box
      }
      if (!ahead.next_step()) ahead_live = ahead.begin_strip();
    };
    for (int i = 0; i < kXBufs; ++i) issue();
    // A quarter warp moves an 8-row x 8-k-group block along its diagonals: lane i takes k group i of row
    // (i + r) & 7, so the eight 16-byte loads (row pitch 256 S bytes) and the eight stores (k-group pitch 128 B) each hit
    // eight different bank groups.  8 quarter warps = 4 blocks (2 row groups x 2 k-group halves) x 2 diagonal sets.
    const int qw = t >> 3, li = t & 7;
    const int mg = (qw >> 1) & 1, kg = (qw & 1) * 8 + li, r0 = (qw >> 2) * 4;
    while (cur.begin_strip()) {
      do {
        const int xb = cur.q % kXBufs;
        if (ok) ok = mbar_wait(x_raw + xb, (cur.q / kXBufs) & 1);
        if (ok && cur.q >= kXBufs) ok = mbar_wait(x_empty + xb, ((cur.q / kXBufs) - 1) & 1);
        if (ok) {
          for (int ks = 0; ks < cur.split; ++ks) {
            const unsigned char* src = xraw + xb * kXRawBytes + ks * (kStepK * 4) + kg * 16;
            unsigned char* dst = xbuf + xb * kXBytes + (ks * 2 + mg) * kXSbo + kg * kXLbo;
            U4 v[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) v[r] = *reinterpret_cast<const U4*>(src + (mg * 8 + ((li + r0 + r) & 7)) * (S * kStepK * 4));
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              U4 hi, lo;
              split_tf32(v[r].x, hi.x, lo.x);
              split_tf32(v[r].y, hi.y, lo.y);
              split_tf32(v[r].z, hi.z, lo.z);
              split_tf32(v[r].w, hi.w, lo.w);
              *reinterpret_cast<U4*>(dst + ((li + r0 + r) & 7) * 16) = hi;
              *reinterpret_cast<U4*>(dst + kXHalfBytes + ((li + r0 + r) & 7) * 16) = lo;
            }
          }
          fence_async_smem();
        }
        asm volatile("bar.sync 2, 64;" ::: "memory");  // both x warps are done with the raw buffer and wrote their share
        if (t == 0) mbar_arrive_cta(x_full + xb);
        issue();
      } while (cur.next_step());
    }
    if (!ok && lane == 0) atomicOr(&g_tc_fault, 4u);
  } else {
    // ------------------------------------------------------------ split warps (+ epilogue)
    const int lq = warp & 3, kh = warp >> 2;  // TMEM lane quarter this warp may touch, k half of a step
    const int c = lq * 32 + lane;             // this thread's TMEM lane
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(lq * 32) << 16);
    const uint32_t a_lane_base = lane_base + kTmemA + kh * (kStepK / 2);
    int strip_i = 0;
    bool ok = true;
    while (cur.begin_strip()) {
      const int qpk = 4 / cur.split;
      const int ks = lq / qpk, uq = lq % qpk;   // this quarter's k range and unit of the strip
      const bool warp_live = uq < cur.units;    // warp-uniform: a quarter without columns writes nothing
      const int col = (cur.unit + uq) * 32 + lane;
      const int split = cur.split;
      const int naccs = min(acc_cols / (16 * S), cur.steps);
      const int pitch = cur.units * 32;  // KN: floats per k row of the tile
      do {
        const int buf = cur.q % kRing, s = cur.q % kStages;
        if (ok) ok = mbar_wait(w_full + buf, (cur.q / kRing) & 1);
        if (ok && cur.q >= kStages) ok = mbar_wait(a_empty + s, ((cur.q / kStages) - 1) & 1);
        if (ok && warp_live) {
          tc_fence_after();
          // NK: this quarter's own tile; KN: the tile of its k range, [64 k][32 u columns], this quarter's columns at 32 uq
          const unsigned char* tile = ring + buf * kStepBytes + (NK ? lq : lq - uq) * kQuarterBytes;
#pragma unroll
          for (int g = 0; g < kStepK / 2 / 16; ++g) {  // 16 k at a time
            uint32_t hi[16], lo[16];
            if (NK) {
              // rows = columns of W, 128 bytes (32 k) each, 16-byte piece p of row r at p ^ (r & 7): the lanes
              // of a warp read the same piece of 32 different rows from all bank groups
              const unsigned char* row = tile + kh * (kQuarterBytes / 2) + lane * 128;
#pragma unroll
              for (int p = 0; p < 4; ++p) {
                const U4 v = *reinterpret_cast<const U4*>(row + (((g * 4 + p) ^ (lane & 7)) << 4));
                split_tf32(v.x, hi[4 * p], lo[4 * p]);
                split_tf32(v.y, hi[4 * p + 1], lo[4 * p + 1]);
                split_tf32(v.z, hi[4 * p + 2], lo[4 * p + 2]);
                split_tf32(v.w, hi[4 * p + 3], lo[4 * p + 3]);
              }
            } else {
              const uint32_t* colp = reinterpret_cast<const uint32_t*>(tile) + (kh * (kStepK / 2) + g * 16) * pitch + uq * 32 + lane;
#pragma unroll
              for (int j = 0; j < 16; ++j) split_tf32(colp[j * pitch], hi[j], lo[j]);
            }
            tmem_st16(a_lane_base + s * kStageCols + g * 16, hi);
            tmem_st16(a_lane_base + s * kStageCols + kStepK + g * 16, lo);
          }
          tmem_wait_st();
          tc_fence_before();
        }
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_cta(a_full + s);
          mbar_arrive_cta(w_empty + buf);
        }
      } while (cur.next_step());
      // ---- epilogue of the strip: warps 0-3 read their own lane quarter of the accumulators
      float sum[16];
      if (warp < 4) {
        if (ok) ok = mbar_wait(acc_full, strip_i & 1);
        if (ok && warp_live) {
          tc_fence_after();
          for (int i = 0; i < issuers; ++i) {
            for (int sel = 0; sel < naccs; ++sel) {
              uint32_t r[16];
              tmem_ld16(lane_base + i * acc_cols + sel * 16 * S + ks * 16, r);  // the 16 columns of this quarter's own k range
#pragma unroll
              for (int m = 0; m < 16; ++m)
                sum[m] = (i == 0 && sel == 0) ? __uint_as_float(r[m]) : __fadd_rn(sum[m], __uint_as_float(r[m]));
            }
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
      const bool owner = warp < 4 && ok && warp_live && ks == 0;  // this thread holds a column's sum over this CTA's K
      if (a.kparts > 1 && warp < 4) {
        if (part != 0) {
          // hand the partial sums to the rank-0 CTA: its inbox must be free (it has read the previous strip's)
          if (ok && strip_i > 0) ok = mbar_wait_cluster(inbox_free, (strip_i - 1) & 1);
          if (owner) {
            const uint32_t dst = cluster_map(inbox + (static_cast<size_t>(part - 1) * 128 + c) * 16, 0u);
#pragma unroll
            for (int m = 0; m < 16; m += 4) cluster_store_f4(dst + m * 4, make_float4(sum[m], sum[m + 1], sum[m + 2], sum[m + 3]));
          }
          cluster_arrive(cluster_map(inbox_full, 0u));  // all 128 epilogue threads arrive, with or without data
        } else {
          if (ok) ok = mbar_wait_cluster(inbox_full, strip_i & 1);
          if (owner && ok) {
            for (int p = 1; p < a.kparts; ++p)  // fixed order: part 0 + 1 + 2 + 3
#pragma unroll
              for (int m = 0; m < 16; ++m) sum[m] = __fadd_rn(sum[m], inbox[(static_cast<size_t>(p - 1) * 128 + c) * 16 + m]);
          }
          asm volatile("bar.sync 3, 128;" ::: "memory");  // warps 0-3: every inbox slot has been read
          // Tell the other parts only when another strip follows: after their last hand-over they may have exited,
          // and an exited CTA's shared memory must not be touched.
          if (threadIdx.x == 0 && cur.unit < cur.unit_end)
            for (int p = 1; p < a.kparts; ++p) cluster_arrive(cluster_map(inbox_free, static_cast<unsigned>(p)));
        }
      }
      if (owner && ok && part == 0 && col < a.n) {
        const float bv = a.bias ? a.bias[col] : 0.0f;
#pragma unroll
        for (int m = 0; m < 16; ++m)
          if (m < a.m) peer_store(a.out, m, col, __fadd_rn(sum[m], bv));
      }
      // all 256 threads meet before the next strip's stages can reach the MMA warps (a_full needs all of them),
      // so the next strip's first MMAs cannot overwrite TMEM (nor its partials the shared buffer) while they are read
      asm volatile("bar.sync 1, 256;" ::: "memory");
      ++strip_i;
    }
    if (!ok && lane == 0) atomicOr(&g_tc_fault, 8u);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kWTma) {
    tc_fence_after();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

// Grid, K split, ring depth and dynamic shared memory of a launch (fills a.total_units, a.ctas, a.split, a.ring).
size_t plan_tc(TcArgs& a, int k, int n) {
  a.total_units = (n + 31) / 32;
  a.ctas = a.total_units < sm_count() ? a.total_units : sm_count();
  const int per_cta = (a.total_units + a.ctas - 1) / a.ctas;
  // Fewer units than half (a quarter) of the SMs: two (four) CTAs of a cluster share every unit along K, so that a
  // narrow projection -- a column shard of a multi-GPU run -- still uses most of the machine.  Clusters of four
  // one-CTA-per-SM blocks fit only 33 at a time on this part, hence the tighter bound for four.
  a.kparts = 1;
  if (a.total_units * 4 <= 132 && sm_count() >= 132) a.kparts = 4;
  else if (a.total_units * 2 <= sm_count()) a.kparts = 2;
  while (a.kparts > 1 && (k % (a.kparts * kStepK) != 0 || k / a.kparts < 4 * kStepK)) a.kparts /= 2;
  a.split = per_cta == 1 ? 4 : (per_cta == 2 ? 2 : 1);
  while (a.split > 1 && (k / a.kparts) % (a.split * kStepK) != 0) a.split /= 2;
  const size_t fixed = kXBufs * static_cast<size_t>(a.split) * (2 * kXHalf1 + kXRaw1) + kRedBytes * a.kparts + 64 * sizeof(uint64_t);
  a.ring = static_cast<int>((220 * 1024 - fixed) / kStepBytes);
  if (a.ring > kMaxRing) a.ring = kMaxRing;
  return a.ring * static_cast<size_t>(kStepBytes) + fixed;
}

template <bool NK>
int launch_tc(const float* x, const float* w, const float* bias, const PeerOut& y, int m, int k, int n, cudaStream_t stream) {
  TcArgs a;
  a.bias = bias, a.out = y, a.m = m, a.k = k, a.n = n;
  const size_t smem = plan_tc(a, k, n);
  CUtensorMap wmaps[4], xmap;
  CUtensorMap& wmap = wmaps[0];
  if (NK) {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(n)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 4};
    const cuuint32_t box[2] = {32, 32};
    if (!encode_tiled(&wmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, w, dims, strides, box, true)) return XDK_ERR_LAUNCH;
    wmaps[1] = wmaps[2] = wmaps[3] = wmap;
  } else {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(k)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(n) * 4};
    for (int u = 1; u <= 4; ++u) {
      const cuuint32_t box[2] = {static_cast<cuuint32_t>(32 * u), kStepK};
      if (!encode_tiled(&wmaps[u - 1], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, w, dims, strides, box, false)) return XDK_ERR_LAUNCH;
    }
  }
  // x[M][K] seen as [row][K part][k range][k inside the range]: one box brings the 64-k step of every range of a part
  const int kper = k / a.kparts / a.split;
  const cuuint64_t xdims[4] = {static_cast<cuuint64_t>(kper), static_cast<cuuint64_t>(a.split), static_cast<cuuint64_t>(a.kparts),
                               static_cast<cuuint64_t>(m)};
  const cuuint64_t xstrides[3] = {static_cast<cuuint64_t>(kper) * 4, static_cast<cuuint64_t>(k / a.kparts) * 4,
                                  static_cast<cuuint64_t>(k) * 4};
  const cuuint32_t xbox[4] = {kStepK, static_cast<cuuint32_t>(a.split), 1, 16};
  if (!encode_tiled(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, x, xdims, xstrides, xbox, false)) return XDK_ERR_LAUNCH;
  auto kernel = gemv_tc_kernel<NK>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (err != cudaSuccess) return note_launch(err);
  return launch(kernel, dim3(a.ctas, a.kparts), dim3(kThreads), smem, stream, static_cast<unsigned>(a.kparts), a, wmaps[0],
                wmaps[1], wmaps[2], wmaps[3], xmap);
}

}  // namespace

bool gemv_tc_eligible(const float* x, const float* w, int64_t m, int64_t k, int64_t n, bool nk) {
  // XDK_GEMV_TC=0 keeps every projection on the CUDA-core kernels (comparison runs)
  static const bool enabled = !(getenv("XDK_GEMV_TC") && getenv("XDK_GEMV_TC")[0] == '0');
  // K <= 16384: the truncating tensor-core accumulation grows with the number of products an accumulator sums
  // (K / 16 each); measured against an FP64 product the relative L2 error is 2.4e-6 at K = 4096 and stays inside
  // the 1e-5 gate up to K = 16384, but reaches 1.5e-5 at K = 32768 -- longer rows stay on the FP32-FMA kernels.
  return enabled && m > 4 && m <= 16 && k % kStepK == 0 && (nk || n % 4 == 0) && aligned16(x) && aligned16(w) &&
         k <= kMaxK && n < (1 << 30) && k * n >= (4LL << 20);
}

int launch_gemv_tc(const float* x, const float* w, const float* bias, const PeerOut& y, int m, int k, int n, bool nk, cudaStream_t stream) {
  return nk ? launch_tc<true>(x, w, bias, y, m, k, n, stream) : launch_tc<false>(x, w, bias, y, m, k, n, stream);
}

bool gemv_tc_plan(int64_t m, int64_t k, int64_t n, bool nk, int32_t out[5]) {
  alignas(16) static const float aligned_dummy[4] = {0, 0, 0, 0};
  if (!gemv_tc_eligible(aligned_dummy, aligned_dummy, m, k, n, nk)) return false;
  TcArgs a;
  const size_t smem = plan_tc(a, static_cast<int>(k), static_cast<int>(n));
  out[0] = a.ctas * a.kparts, out[1] = a.split, out[2] = a.ring, out[3] = static_cast<int32_t>(smem), out[4] = a.total_units;
  return true;
}

unsigned gemv_tc_fault_word() {
  unsigned v = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_fault, sizeof(v)) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0x80000000u;
  }
  return v;
}

}  // namespace xdk
