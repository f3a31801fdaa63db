// FP32 small-M projection on the 5th-generation tensor cores (tcgen05, kind::tf32) with FP32-grade accuracy.
//
// y[M, N] = x[M, K] . W + bias for 4 < M <= 16.  On CUDA cores this shape is bound by FP32 operand delivery
// (16 rows of x against every weight), not by HBM; the tensor cores have the throughput, but a TF32 product keeps
// only 11 significant bits of each operand.  So every operand is split into two TF32 numbers,
//     v = hi + lo,   hi = v with the low 13 mantissa bits cleared,   lo = v - hi  (exact in FP32),
// and the product is formed as hi.hi + hi.lo + lo.hi with FP32 accumulation in TMEM.  The dropped lo.lo term and
// the bits of lo the tensor core ignores are below 2^-21 relative per product.  The accumulation inside the
// tensor core may truncate instead of rounding; to keep that bias small the sum is spread over several
// accumulators (one or more per MMA issuer, the hi.lo products in columns of their own) that are added in FP32 in a
// fixed order at the end, so results are deterministic.  Measured against an FP64 product the relative L2 error
// stays inside the 1e-5 gate of the projection up to K = 16384; callers that need strict FP32 FMA arithmetic pass
// XDK_STRICT_FP32 and get the CUDA-core kernels instead.
//
// Layout of the work (same scheme as the W4A16 tcgen05 kernel): operands are swapped so that the UMMA "M"
// dimension (128 TMEM lanes) carries output columns, A = W (split) in tensor memory, B = x^T (split) in shared
// memory.  The hi and lo images of x sit one after the other at the same row-group pitch, so one operand
// descriptor covers [x_hi | x_lo] and a k block takes two MMAs instead of three:
//     D[128 lanes x 32 S] += W_hi[128 x 8 k] * [x_hi | x_lo][8 k x 32 S]      (hi.hi and hi.lo, side by side)
//     D[128 lanes x 16 S] += W_lo[128 x 8 k] * x_hi[8 k x 16 S]               (lo.hi, onto the hi.hi columns)
// and the epilogue adds the two halves.  One persistent CTA per SM owns an evenly dealt range of 32-column units
// and walks it in strips of <= 4 units.  K can be split two ways: S ways over the TMEM lane quarters of a CTA
// (narrow strips; the S partial sums meet in shared memory) and over the 2, 4 or 8 CTAs of a thread-block cluster
// (every CTA walks the same strips over its own part of K, the parts store their partial sums into the rank-0
// CTA's shared memory -- distributed shared memory, mbarrier hand-off with bounded waits -- and rank 0 adds them
// in rank order); plan_tc weighs the combinations.  Sums are added in a fixed order everywhere: deterministic.
//   TMA warps (4)      : one warp per TMEM lane quarter: the W tile of a 64-k step (NK: two 128-byte swizzled
//                        [32 columns][32 k] boxes per quarter; KN: one [64 k][32 u columns] box per k range, u = units
//                        of the strip, so that HBM sees runs of up to 512 bytes) into a ring of step buffers
//   x warps (2)        : one lane issues one TMA box per step ([16 rows][S k ranges][64 k]); both warps split every
//                        16-byte unit into hi and lo and move it to its place in the two K-major core-matrix images
//   split warps (8)    : thread = one TMEM lane = one output column; warp w owns lane quarter w % 4 and k half
//                        w / 4 of every step: shared loads -> hi/lo -> tcgen05.st into the stage's hi and lo columns
//   MMA warps (4)      : the 8 k blocks of a step are dealt round-robin to the 4 issuers, each with its own
//                        accumulators (all MMAs of a step onto one of them, steps alternating between them)
//   split warps 0-3    : epilogue -- tcgen05.ld of the accumulators, fixed-order sum, bias, FP32 store
// The TMA and MMA roles run their loops with the whole warp (waits included) and issue under elect.sync: the same
// loop run by lane 0 alone got a tcgen05.mma out only every ~120 ns, the elected form every ~70 ns.  Ring slots and
// parities are kept by increments (RingPos): a step is a chain TMA -> split -> MMA -> (stage free) -> split in which
// every role's own per-step instructions are the cost -- a tcgen05.st is ~125 ns per warp whatever its width, a
// division in a one-thread role 0.1 us -- and that chain, not HBM, sets the step time (a run without any W traffic
// took as long).  A third A stage, a third x buffer, sixteen split warps and 32-column stores were each measured:
// no gain, so two stages, two x buffers (buffer s and stage s share their "MMAs done" barrier) and eight warps.
// The kernel's time also moves by several per cent with how the compiler schedules the roles, so the switches of
// those comparisons (XDK_TC_MMA3, XDK_TC_NACCS, XDK_TC_ROT, XDK_TC_SLOT; defaults = the fastest measured) stayed in.
// TMEM columns (512): accumulators first -- 64 per issuer, 32 S per accumulator (hi.hi + lo.hi | hi.lo) -- then
// stage s at 256 + 128 s: 64 hi columns, 64 lo.
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
constexpr int kMaxK = 16384;                    // largest K the path takes
// The tensor core's accumulation truncates, so the error of a sum grows with the number of products one accumulator
// adds: measured against FP64 with the eight accumulators a CTA has, zero-mean operands give a relative L2 error of
// 2.9e-6 at 4096 k per CTA and 1.0e-5 at 16384; all-positive operands (the worst case) 7.6e-6 and 3.0e-5.  A CTA
// therefore never sums more than 4096 k: longer rows are split over the CTAs of a cluster (whose partial sums are
// added in FP32 with rounding) or, when K does not divide, left to the FP32-FMA kernels.
constexpr int kMaxKPerCta = 4096;
constexpr int kMaxRing = 8;                     // W step buffers: as many as shared memory leaves (plan.ring)
constexpr int kQuarterBytes = 32 * kStepK * 4;  // one lane quarter's tile: 32 columns x 64 k
constexpr int kStepBytes = 4 * kQuarterBytes;
constexpr int kStages = 2;                      // A stages in TMEM (a third one measured no faster)
constexpr int kStageCols = 2 * kStepK;          // hi columns then lo columns
constexpr int kMaxIssuers = 4;
constexpr int kTmemCols = 512;                  // accumulators first (256 columns, 64 per issuer), then the stages
constexpr int kTmemA = kTmemCols - kStages * kStageCols;
constexpr int kXLbo = 128, kXSbo = (kStepK / 4) * kXLbo;  // x image: [row group of 8][16 k groups][8 rows x 16 B]
constexpr int kXHalf1 = 2 * kXSbo;              // hi (or lo) image of one k range: 16 rows
constexpr int kXRaw1 = 16 * kStepK * 4;         // one k range of [16 rows][64 k] as TMA lands it
constexpr int kXBufs = kStages;                 // x steps in flight: buffer s serves A stage s, one barrier frees both
constexpr int kRedBytes = 128 * 16 * 4;         // k-range partials: [lane][16] floats
constexpr int kMaxParts = 8;                    // CTAs of a cluster sharing a strip along K (portable cluster size)
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
  int kparts; // CTAs of a cluster that share every strip, each walking K / kparts (1, 2, 4, 8); grid = (ctas, kparts)
  int wide;   // 1: W_hi meets [x_hi | x_lo] in one MMA of 32 S columns (2 MMAs per k block); 0: three MMAs of 16 S
  int max_accs;
  int rotate;     // 1: every CTA starts its k loop at another step (no two CTAs ask L2 for the same x lines at once)
  int tight_ring; // 1: a CTA whose strips are narrower than 128 columns cuts the ring into smaller, more slots
};


__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&r)[16]) {  // no wait: see tmem_ld_wait16
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
// Waits for every tcgen05.ld of this thread; the registers pass through the statement so that no use of them can
// be scheduled before the wait.
__device__ __forceinline__ void tmem_ld_wait16(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :: "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

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
  const int S = a.split;
  const int issuers = kMaxIssuers, acc_cols = kTmemA / issuers;
  const int acc_w = a.wide ? 32 : 16;  // columns of an accumulator per k range: [hi.hi + lo.hi | hi.lo] or one sum
  const int kXHalfBytes = S * kXHalf1, kXBytes = 2 * kXHalfBytes, kXRawBytes = S * kXRaw1;
  unsigned char* ring = smem_raw;                            // [a.ring][kStepBytes], re-cut below
  unsigned char* xbuf = ring + a.ring * kStepBytes;          // [kXBufs][hi image | lo image], 16 S rows each
  unsigned char* xraw = xbuf + kXBufs * kXBytes;             // [kXBufs][16 rows][S k ranges][64 k]
  // k-range partials of this CTA, [row quad][lane] float4 (a thread's 16 sums sit 2 KB apart: conflict-free)
  float4* red = reinterpret_cast<float4*>(xraw + kXBufs * kXRawBytes);
  // partial sums of the other CTAs of the cluster land here (in the rank-0 CTA): [part - 1][row quad][lane] float4
  float4* inbox = red + kRedBytes / sizeof(float4);
  uint64_t* bars = reinterpret_cast<uint64_t*>(inbox + (a.kparts - 1) * (kRedBytes / sizeof(float4)));
  uint64_t* w_full = bars;                 // [kMaxRing] TMA bytes of a W step landed
  uint64_t* w_empty = w_full + kMaxRing;   // [kMaxRing] the 8 split warps are done with the step
  uint64_t* a_full = w_empty + kMaxRing;   // [kStages] the 8 split warps wrote the stage to TMEM
  uint64_t* mma_done = a_full + kStages;   // [kStages] every issuer's MMAs on the stage (and its x images) completed
  uint64_t* x_raw = mma_done + kStages;    // [kXBufs]  TMA bytes of an x step landed
  uint64_t* x_full = x_raw + kXBufs;       // [kXBufs]  the x warps wrote both operand images
  uint64_t* acc_full = x_full + kXBufs;    // [1]
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
  // The ring holds a.ring steps of 128 columns.  A CTA whose widest strip (its first) has fewer columns needs less
  // per step and cuts the same bytes into more slots: more W in flight against the 3-4 us a load takes under load.
  const int widest = min(4, cur.unit_end - cur.unit);
  const int slot_bytes = (a.tight_ring && S == 1 && widest > 0) ? widest * kQuarterBytes : kStepBytes;
  const int kRing = min(kMaxRing, a.ring * kStepBytes / slot_bytes);
  // first k step of this CTA's loop over a strip (taken modulo the strip's steps)
  const int rot_seed = a.rotate ? static_cast<int>(blockIdx.x) * 5 + part * 3 : 0;

  if (warp == 0) {  // one barrier per lane
    if (lane < kRing) {
      mbar_init(w_full + lane, 4);   // one arrival (with its bytes) per TMA warp
      mbar_init(w_empty + lane, 8);
    }
    if (lane < kStages) {
      mbar_init(x_raw + lane, 1);
      mbar_init(x_full + lane, 1);
      mbar_init(a_full + lane, 8);
      mbar_init(mma_done + lane, issuers);
    }
    if (lane == 0) {
      mbar_init(acc_full, issuers);
      mbar_init(inbox_full, 128 * (a.kparts - 1) > 0 ? 128 * (a.kparts - 1) : 1);
      mbar_init(inbox_free, 1);
    }
    mbar_fence_init();
  } else if (warp >= kWTma && warp < kWX0 && lane == 0) {
    prefetch_tensormap(warp == kWTma ? &wmap : (warp == kWTma + 1 ? &wmap2 : (warp == kWTma + 2 ? &wmap3 : &wmap4)));
  } else if (warp == kWX0 && lane == 0) {
    prefetch_tensormap(&xmap);
  }
  __syncthreads();  // the barriers exist: the TMA and x warps start their loads
  // Every CTA of a cluster must know that its peers' barriers exist before it arrives on them (the first remote
  // access is in the epilogue).  Everybody arrives here; each warp waits where it has nothing better to do.
  const bool clustered = a.kparts > 1;
  if (clustered) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  uint32_t tmem_base = 0;
  if (warp < kWTma || warp >= kWMma0) {  // the warps that touch tensor memory: split warps and MMA warps
    if (warp == kWMma0) tmem_alloc<kTmemCols>(tmem_slot);
    tc_fence_before();
    asm volatile("bar.sync 4, %0;" ::"n"((kWTma + kMaxIssuers) * 32) : "memory");
    tc_fence_after();
    tmem_base = *tmem_slot;
    if (clustered) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }

  if (warp >= kWTma && warp < kWX0) {
    // ------------------------------------------------------------ TMA producers: W tiles, one lane quarter each
    {  // the whole warp runs the loop (waits included), one elected lane issues
      const int lq = warp - kWTma;
      bool ok = true;
      RingPos w;
      while (ok && cur.begin_strip()) {
        const int qpk = 4 / cur.split;  // lane quarters per k range = units the strip can hold
        const bool live = lq % qpk < cur.units;
        const int col0 = (cur.unit + lq % qpk) * 32, k_range0 = (lq / qpk) * cur.kper;
        int kk = rot_seed % cur.steps;  // the step this CTA walks now: kk, kk + 1, ..., steps - 1, 0, ...
        do {
          const int buf = w.slot;
          ok = __all_sync(0xffffffffu, mbar_wait(w_empty + buf, w.parity ^ 1u));
          if (!ok) break;
          w.advance(kRing);
          const int k0 = k_base + k_range0 + kk * kStepK;
          kk = kk + 1 == cur.steps ? 0 : kk + 1;
          if (elect_one()) {
            unsigned char* dst = ring + buf * slot_bytes + lq * kQuarterBytes;
            if (NK) {  // two [32 columns][32 k] boxes, 128-byte rows, swizzled
              if (!live) {
                mbar_arrive_cta(w_full + buf);
              } else {
                mbar_expect_tx(w_full + buf, static_cast<unsigned>(kQuarterBytes));
                tma_box_2d(dst, &wmap, k0, col0, w_full + buf);
                tma_box_2d(dst + kQuarterBytes / 2, &wmap, k0 + 32, col0, w_full + buf);
              }
            } else {   // the first quarter of each k range fetches [64 k][32 u columns] for all its quarters
              if (lq % qpk != 0) {
                mbar_arrive_cta(w_full + buf);
              } else {
                mbar_expect_tx(w_full + buf, static_cast<unsigned>(cur.units * kQuarterBytes));
                const CUtensorMap* map = cur.units == 1 ? &wmap : (cur.units == 2 ? &wmap2 : (cur.units == 3 ? &wmap3 : &wmap4));
                tma_box_2d(dst, map, col0, k0, w_full + buf);
              }
            }
          }
          __syncwarp();
        } while (cur.next_step());
      }
      if (!ok && lane == 0) atomicOr(&g_tc_fault, 1u);
    }
    if (clustered) asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
  } else if (warp >= kWMma0) {
    // ------------------------------------------------------------ MMA issuers
    if (warp - kWMma0 < issuers) {  // the whole warp runs the loop; one elected lane issues
      const int issuer = warp - kWMma0;
      const uint64_t xd0 = umma_desc(smem_u32(xbuf), kXLbo, kXSbo);
      const uint32_t xd_lo = static_cast<uint32_t>(xd0), xd_hi = static_cast<uint32_t>(xd0 >> 32);
      bool ok = true;
      RingPos st;
      while (ok && cur.begin_strip()) {
        const uint32_t idesc = umma_idesc(16 * cur.split, 2u), idesc_wide = umma_idesc(32 * cur.split, 2u);
        const int naccs = min(min(acc_cols / (acc_w * S), cur.steps), a.max_accs);
        do {
          const int s = st.slot, xb = s;
          ok = __all_sync(0xffffffffu, mbar_wait(x_full + xb, st.parity) && mbar_wait(a_full + s, st.parity));
          if (!ok) break;
          st.advance(kStages);
          tc_fence_after();
          // All MMAs of a step go to one accumulator, steps rotate over the accumulators: measured, an issuer that
          // changes accumulator from one MMA to the next loses 50-80 cycles per MMA.
          const int nj = kStepK / 8 / issuers;  // k blocks of this issuer per step: issuer, issuer + issuers, ...
          const uint32_t acc = tmem_base + issuer * acc_cols + (cur.kc % naccs) * acc_w * S;
          const bool fresh = cur.kc < naccs;  // first step that touches this accumulator in the strip
          const uint32_t a_hi = tmem_base + kTmemA + s * kStageCols + issuer * 8;
          const uint32_t x_lo = xd_lo + ((xb * kXBytes + issuer * 2 * kXLbo) >> 4);
          if (elect_one()) {
          for (int j = 0; j < nj; ++j) {
            uint64_t b_hi, b_lo;
            const uint32_t off = (j * issuers * 2 * kXLbo) >> 4;
            asm("mov.b64 %0, {%1, %2};" : "=l"(b_hi) : "r"(x_lo + off), "r"(xd_hi));
            asm("mov.b64 %0, {%1, %2};" : "=l"(b_lo) : "r"(x_lo + off + (kXHalfBytes >> 4)), "r"(xd_hi));
            const uint32_t ah = a_hi + j * issuers * 8;
            if (a.wide) {  // the lo image follows the hi image at the same row-group pitch: one operand of 32 S rows
              umma_tf32_ta(acc, ah, b_hi, idesc_wide, !(fresh && j == 0));
              umma_tf32_ta(acc, ah + kStepK, b_hi, idesc, true);
            } else {
              umma_tf32_ta(acc, ah, b_hi, idesc, !(fresh && j == 0));
              umma_tf32_ta(acc, ah, b_lo, idesc, true);
              umma_tf32_ta(acc, ah + kStepK, b_hi, idesc, true);
            }
          }
          umma_commit(mma_done + s);
          }
          __syncwarp();
        } while (cur.next_step());
        if (ok && elect_one()) umma_commit(acc_full);
        __syncwarp();
      }
      if (!ok && lane == 0) atomicOr(&g_tc_fault, 2u);
    }
  } else if (warp >= kWX0) {  // the two warps between the TMA warps and the MMA warps
    // ------------------------------------------------------------ x warps
    const int t = threadIdx.x - kWX0 * 32;  // 0 .. 63
    bool ok = true;
    UmmaCursor ahead = cur;  // issues the loads, kXBufs steps in front of `cur`
    bool ahead_live = ahead.begin_strip();
    RingPos xi, xs;          // of the load being issued, of the step being transformed
    int xkk = ahead_live ? rot_seed % ahead.steps : 0;
    auto issue = [&]() {  // raw buffer xi.slot is free: its last readers passed the x-warp barrier
      if (!ahead_live) return;
      if (t == 0) {
        const int xb = xi.slot;
        mbar_expect_tx(x_raw + xb, static_cast<unsigned>(kXRawBytes));  // rows >= M are out of range: zero-filled, still counted
        tma_box_4d(xraw + xb * kXRawBytes, &xmap, xkk * kStepK, 0, part, 0, x_raw + xb);  // all k ranges in one box
      }
      xi.advance(kXBufs);
      xkk = xkk + 1 == ahead.steps ? 0 : xkk + 1;
      if (!ahead.next_step()) {
        ahead_live = ahead.begin_strip();
        if (ahead_live) xkk = rot_seed % ahead.steps;
      }
    };
    for (int i = 0; i < kXBufs; ++i) issue();
    // A quarter warp moves an 8-row x 8-k-group block along its diagonals: lane i takes k group i of row
    // (i + r) & 7, so the eight 16-byte loads (row pitch 256 S bytes) and the eight stores (k-group pitch 128 B) each hit
    // eight different bank groups.  8 quarter warps = 4 blocks (2 row groups x 2 k-group halves) x 2 diagonal sets.
    const int qw = t >> 3, li = t & 7;
    const int mg = (qw >> 1) & 1, kg = (qw & 1) * 8 + li, r0 = (qw >> 2) * 4;
    while (cur.begin_strip()) {
      do {
        const int xb = xs.slot;
        if (ok) ok = mbar_wait(x_raw + xb, xs.parity);
        if (ok) ok = mbar_wait(mma_done + xb, xs.parity ^ 1u);  // the MMAs that read these images two steps ago
        xs.advance(kXBufs);
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
    if (clustered) asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
  } else {
    // ------------------------------------------------------------ split warps (+ epilogue)
    const int lq = warp & 3, kh = warp >> 2;  // TMEM lane quarter this warp may touch, k half of a step
    const int c = lq * 32 + lane;             // this thread's TMEM lane
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(lq * 32) << 16);
    const uint32_t a_lane_base = lane_base + kTmemA + kh * (kStepK / 2);
    int strip_i = 0;
    bool ok = true;
    RingPos w, st;
    while (cur.begin_strip()) {
      const int qpk = 4 / cur.split;
      const int ks = lq / qpk, uq = lq % qpk;   // this quarter's k range and unit of the strip
      const bool warp_live = uq < cur.units;    // warp-uniform: a quarter without columns writes nothing
      const int col = (cur.unit + uq) * 32 + lane;
      const int split = cur.split;
      const int naccs = min(min(acc_cols / (acc_w * S), cur.steps), a.max_accs);
      const int pitch = cur.units * 32;  // KN: floats per k row of the tile
      do {
        const int buf = w.slot, s = st.slot;
        if (ok) ok = mbar_wait(w_full + buf, w.parity);
        if (ok) ok = mbar_wait(mma_done + s, st.parity ^ 1u);
        w.advance(kRing), st.advance(kStages);
        if (ok && warp_live) {
          tc_fence_after();
          // NK: this quarter's own tile; KN: the tile of its k range, [64 k][32 u columns], this quarter's columns at 32 uq
          const unsigned char* tile = ring + buf * slot_bytes + (NK ? lq : lq - uq) * kQuarterBytes;
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
              // the tile's row pitch follows the strip's width; one copy of the sixteen loads per width, so that their
              // offsets are immediates instead of an address computation per load
              const uint32_t* colp = reinterpret_cast<const uint32_t*>(tile) + (kh * (kStepK / 2) + g * 16) * pitch + uq * 32 + lane;
              if (pitch == 96) {
#pragma unroll
                for (int j = 0; j < 16; ++j) split_tf32(colp[j * 96], hi[j], lo[j]);
              } else if (pitch == 128) {
#pragma unroll
                for (int j = 0; j < 16; ++j) split_tf32(colp[j * 128], hi[j], lo[j]);
              } else if (pitch == 32) {
#pragma unroll
                for (int j = 0; j < 16; ++j) split_tf32(colp[j * 32], hi[j], lo[j]);
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) split_tf32(colp[j * 64], hi[j], lo[j]);
              }
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
      float bias_v = 0.0f;
      const bool stores = warp < 4 && warp_live && ks == 0 && part == 0 && col < a.n;  // this thread writes a column of y
      if (stores && a.bias) bias_v = __ldg(a.bias + col);  // in flight while the last MMAs complete
      if (warp < 4) {
        if (ok) ok = mbar_wait(acc_full, strip_i & 1);
        if (ok && warp_live) {
          tc_fence_after();
          // one accumulator per round: its loads (hi.hi + lo.hi columns, and hi.lo columns in the wide form) go out
          // together and are waited for once; fixed order of additions
          for (int i = 0; i < issuers; ++i) {
            for (int sel = 0; sel < naccs; ++sel) {
              uint32_t r0[16], r1[16];
              const uint32_t t0 = lane_base + i * acc_cols + sel * acc_w * S + ks * 16;
              tmem_ld16_issue(t0, r0);
              if (a.wide) tmem_ld16_issue(t0 + 16 * S, r1);
              tmem_ld_wait16(r0);
              if (a.wide) tmem_ld_wait16(r1);
#pragma unroll
              for (int m = 0; m < 16; ++m) {
                float v = __uint_as_float(r0[m]);
                if (a.wide) v = __fadd_rn(v, __uint_as_float(r1[m]));
                sum[m] = (i == 0 && sel == 0) ? v : __fadd_rn(sum[m], v);
              }
            }
          }
          tc_fence_before();
          if (split > 1) {
#pragma unroll
            for (int m = 0; m < 16; m += 4) red[(m >> 2) * 128 + c] = make_float4(sum[m], sum[m + 1], sum[m + 2], sum[m + 3]);
          }
        }
      }
      if (split > 1) {
        asm volatile("bar.sync 1, 256;" ::: "memory");  // strip-uniform: the k-range partials are in shared memory
        if (warp < 4 && ok && warp_live && ks == 0) {
          for (int j = 1; j < split; ++j)  // fixed order: k range 0 + 1 + 2 + 3
#pragma unroll
            for (int m = 0; m < 16; m += 4) {
              const float4 v = red[(m >> 2) * 128 + c + j * qpk * 32];
              sum[m] = __fadd_rn(sum[m], v.x), sum[m + 1] = __fadd_rn(sum[m + 1], v.y);
              sum[m + 2] = __fadd_rn(sum[m + 2], v.z), sum[m + 3] = __fadd_rn(sum[m + 3], v.w);
            }
        }
      }
      const bool owner = warp < 4 && ok && warp_live && ks == 0;  // this thread holds a column's sum over this CTA's K
      if (a.kparts > 1 && warp < 4) {
        if (part != 0) {
          // hand the partial sums to the rank-0 CTA: its inbox must be free (it has read the previous strip's)
          if (ok && strip_i > 0) ok = mbar_wait_cluster(inbox_free, (strip_i - 1) & 1);
          if (owner) {
            const uint32_t dst = cluster_map(inbox + (part - 1) * 512 + c, 0u);
#pragma unroll
            for (int m = 0; m < 16; m += 4)
              cluster_store_f4(dst + (m >> 2) * 128 * 16, make_float4(sum[m], sum[m + 1], sum[m + 2], sum[m + 3]));
          }
          cluster_arrive(cluster_map(inbox_full, 0u));  // all 128 epilogue threads arrive, with or without data
        } else {
          if (ok) ok = mbar_wait_cluster(inbox_full, strip_i & 1);
          if (owner && ok) {
            for (int p = 1; p < a.kparts; ++p)  // fixed order: part 0 + 1 + 2 + ...
#pragma unroll
              for (int m = 0; m < 16; m += 4) {
                const float4 v = inbox[(p - 1) * 512 + (m >> 2) * 128 + c];
                sum[m] = __fadd_rn(sum[m], v.x), sum[m + 1] = __fadd_rn(sum[m + 1], v.y);
                sum[m + 2] = __fadd_rn(sum[m + 2], v.z), sum[m + 3] = __fadd_rn(sum[m + 3], v.w);
              }
          }
          asm volatile("bar.sync 3, 128;" ::: "memory");  // warps 0-3: every inbox slot has been read
          // Tell the other parts only when another strip follows: after their last hand-over they may have exited,
          // and an exited CTA's shared memory must not be touched.
          if (threadIdx.x == 0 && cur.unit < cur.unit_end)
            for (int p = 1; p < a.kparts; ++p) cluster_arrive(cluster_map(inbox_free, static_cast<unsigned>(p)));
        }
      }
      if (stores && ok) {
#pragma unroll
        for (int m = 0; m < 16; ++m)
          if (m < a.m) peer_store(a.out, m, col, __fadd_rn(sum[m], bias_v));
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
  if (warp == kWMma0) {
    tc_fence_after();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

// How many clusters of `parts` one-CTA-per-SM blocks the device runs at once.  A cluster must sit inside one GPC, so
// this is less than SMs / parts; the driver is asked once per cluster size, and without a device (plan
// introspection on a build host) the answer defaults to what a 148-SM B200 gives.
int resident_clusters(int parts) {
  static int cached[kMaxParts + 1] = {};
  if (parts == 1) return sm_count();
  if (cached[parts] > 0) return cached[parts];
  const int sms = sm_count();
  int fit = parts == 2 ? sms / 2 : (parts == 4 ? (sms >= 132 ? 33 : sms / 6) : (sms >= 132 ? 16 : sms / 12));
  int devices = 0;
  if (cudaGetDeviceCount(&devices) == cudaSuccess && devices > 0) {
    auto kernel = gemv_tc_kernel<false>;
    const int smem = 220 * 1024;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 1, attr.val.clusterDim.y = static_cast<unsigned>(parts), attr.val.clusterDim.z = 1;
    cfg.gridDim = dim3(sms / parts, parts), cfg.blockDim = dim3(kThreads), cfg.dynamicSmemBytes = smem, cfg.attrs = &attr, cfg.numAttrs = 1;
    int n = 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
        cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) == cudaSuccess && n > 0)
      fit = n < sms / parts ? n : sms / parts;
  }
  (void)cudaGetLastError();
  if (fit < 1) fit = 1;
  return cached[parts] = fit;
}

// Grid, K splits, ring depth and dynamic shared memory of a launch (fills a.total_units, a.ctas, a.split, a.kparts,
// a.ring).  K can be split two ways: over the TMEM lane quarters of a CTA (S: cheap to add up, but a 64-k step then
// carries S x 16 operand rows and takes ~0.62 / 0.85 / 1.3 us of MMA issue for S = 1 / 2 / 4) and over the CTAs of a
// cluster (parts: full-rate steps, one hand-over per strip through distributed shared memory).  The plan minimises
// the modelled time: the busiest CTA's steps x step time, or the time HBM needs for W if that is longer, plus the
// hand-overs.
size_t plan_tc(TcArgs& a, int k, int n) {
  a.total_units = (n + 31) / 32;
  const float step_us[5] = {0.0f, 0.62f, 0.85f, 0.0f, 1.3f};
  const float hbm_us = static_cast<float>(k) * static_cast<float>(n) * 4.0f / 6.0e6f;
  static const bool three = getenv("XDK_TC_MMA3") && getenv("XDK_TC_MMA3")[0] == '1';
  a.wide = three ? 0 : 1;
  const int acc_w = a.wide ? 32 : 16;
  const int max_split = kTmemA / kMaxIssuers / acc_w;  // an accumulator must fit an issuer's columns
  float best = 1e30f;
  a.kparts = 0, a.split = 1, a.ctas = 0;
  for (int parts = 1; parts <= kMaxParts; parts *= 2) {
    if (k % (parts * kStepK) != 0 || (parts > 1 && k / parts < 4 * kStepK)) continue;
    if (k / parts > kMaxKPerCta) continue;  // accuracy: see kMaxKPerCta
    for (int split = 1; split <= max_split; split *= 2) {
      if ((k / parts) % (split * kStepK) != 0) continue;
      const size_t other = kXBufs * static_cast<size_t>(split) * (2 * kXHalf1 + kXRaw1) + kRedBytes * parts + 64 * sizeof(uint64_t);
      if (other + 3 * kStepBytes > 220 * 1024) continue;  // the W ring needs three steps in flight
      const int upc = 4 / split;  // units a strip holds
      int ctas = resident_clusters(parts);
      if (ctas > a.total_units) ctas = a.total_units;
      const int units = (a.total_units + ctas - 1) / ctas;  // of the busiest CTA
      const int strips = (units + upc - 1) / upc;
      float cost = strips * (k / parts / split / kStepK) * step_us[split];
      if (cost < hbm_us) cost = hbm_us;
      if (parts > 1) cost += 0.7f + 0.3f * strips + 0.05f * parts;
      if (cost < best - 1e-3f) best = cost, a.kparts = parts, a.split = split, a.ctas = ctas;
    }
  }
  if (a.kparts == 0) return 0;  // no admissible split of this K
  static const int forced_accs = getenv("XDK_TC_NACCS") ? atoi(getenv("XDK_TC_NACCS")) : 0;
  a.max_accs = forced_accs > 0 ? forced_accs : 64;
  static const bool no_rotate = getenv("XDK_TC_ROT") && getenv("XDK_TC_ROT")[0] == '0';
  static const bool no_tight = getenv("XDK_TC_SLOT") && getenv("XDK_TC_SLOT")[0] == '0';
  a.rotate = no_rotate ? 0 : 1, a.tight_ring = no_tight ? 0 : 1;
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
  if (smem == 0) return XDK_ERR_LIMIT;
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
  // the shape must also have a launch plan: a K split that keeps every CTA's share of K inside kMaxKPerCta
  if (!(enabled && m > 4 && m <= 16 && k % kStepK == 0 && (nk || n % 4 == 0) && aligned16(x) && aligned16(w) && k <= kMaxK &&
        n < (1 << 30) && k * n >= (4LL << 20)))
    return false;
  TcArgs a;
  return plan_tc(a, static_cast<int>(k), static_cast<int>(n)) != 0;
}

int launch_gemv_tc(const float* x, const float* w, const float* bias, const PeerOut& y, int m, int k, int n, bool nk, cudaStream_t stream) {
  return nk ? launch_tc<true>(x, w, bias, y, m, k, n, stream) : launch_tc<false>(x, w, bias, y, m, k, n, stream);
}

int gemv_tc_plan(int64_t m, int64_t k, int64_t n, bool nk, int32_t out[5]) {
  alignas(16) static const float aligned_dummy[4] = {0, 0, 0, 0};
  if (!gemv_tc_eligible(aligned_dummy, aligned_dummy, m, k, n, nk)) return 0;
  TcArgs a;
  const size_t smem = plan_tc(a, static_cast<int>(k), static_cast<int>(n));
  out[0] = a.ctas * a.kparts, out[1] = a.split, out[2] = a.ring, out[3] = static_cast<int32_t>(smem), out[4] = a.total_units;
  return a.kparts;
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
