// tcgen05 / TMEM / TMA building blocks shared by the kernels whose contraction runs on the 5th-generation
// tensor cores with the A operand in tensor memory (w4a16.cu, gemv_tc.cu).
#pragma once

#include "common.cuh"

namespace xdk {

// Shared-memory matrix descriptor, K-major, no swizzle: core matrices of 8 rows x 16 bytes; `lbo` = bytes
// between core matrices adjacent in K, `sbo` = bytes between 8-row groups.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, int lbo, int sbo) {
  return static_cast<uint64_t>((smem_addr >> 4) & 0x3fff) | (static_cast<uint64_t>((lbo >> 4) & 0x3fff) << 16) |
         (static_cast<uint64_t>((sbo >> 4) & 0x3fff) << 32) | (1ull << 46);  // version 1
}
// Instruction descriptor: FP32 accumulator, both operands K-major, M = 128, N = `n`; `ab_format`: 0 = F16, 2 = TF32.
__device__ __forceinline__ uint32_t umma_idesc(int n, uint32_t ab_format) {
  return (1u << 4) | (ab_format << 7) | (ab_format << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (8u << 24);
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
__device__ __forceinline__ void umma_tf32_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}
// True in exactly one lane of a converged warp.  A role whose loop the whole warp runs (waits included) and that
// issues its tcgen05.mma / TMA instructions under this predicate keeps its operands warp-uniform; the same loop
// run by `if (lane == 0)` alone issued each tcgen05.mma ~120 ns after the previous one.
__device__ __forceinline__ bool elect_one() {
  uint32_t is_elected;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(is_elected));
  return is_elected != 0;
}
// 32 lanes (the warp's TMEM lane quarter) x 16 consecutive 32-bit columns
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// 32 lanes x 32 consecutive columns.  A tcgen05.st costs the issuing warp ~125 ns whatever its width (measured:
// x8, x16 and x32 alike), so the widest store the registers allow is the cheapest.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
template <int COLS>
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_smem) {  // one warp; writes the base address to *slot_smem
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_smem)), "n"(COLS) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <int COLS>
__device__ __forceinline__ void tmem_dealloc(uint32_t base) {  // the warp that allocated
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "n"(COLS) : "memory");
}
// mbarrier arrive (count 1) once every tcgen05.mma this thread issued before has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_cta(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One TMA op: the 2-D box at element coordinates (c0, c1) of `map` -> dense rows at dst; completes on `bar`.
__device__ __forceinline__ void tma_box_2d(void* dst_smem, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst_smem)),
      "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tma_box_3d(void* dst_smem, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          smem_u32(dst_smem)),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tma_box_4d(void* dst_smem, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
          smem_u32(dst_smem)),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
      : "memory");
}

// ---- hand-off between the CTAs of a thread-block cluster through distributed shared memory -------------------
// Address of `local` (a shared-memory address of this CTA) in the CTA of rank `cta_rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_map(const void* local, unsigned cta_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(cta_rank));
  return remote;
}
__device__ __forceinline__ void cluster_store_f4(uint32_t remote, float4 v) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// Arrive (count 1) on an mbarrier of another CTA of the cluster; orders this thread's earlier remote stores before it.
__device__ __forceinline__ void cluster_arrive(uint32_t remote_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
// Bounded wait on an mbarrier of THIS CTA that other CTAs of the cluster arrive on (acquire at cluster scope).
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, unsigned parity, uint64_t budget_ns = 20000000ull) {
  const uint32_t addr = smem_u32(bar);
  uint64_t t0 = 0;
  for (unsigned i = 0;; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if ((i & 15u) == 15u) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_ns) return false;
    }
  }
}

// Position in a ring of `depth` buffers guarded by full/empty mbarriers: the slot and the parity a consumer waits
// for on the slot's "full" barrier; a producer waits for parity ^ 1 on the "empty" barrier (which a fresh barrier
// already satisfies).  Kept by increments: the roles' loops are latency chains, a division per step shows.
struct RingPos {
  int slot = 0;
  uint32_t parity = 0;
  __device__ __forceinline__ void advance(int depth) {
    if (++slot == depth) slot = 0, parity ^= 1u;
  }
};

// The K split of a strip of `units` 32-column units: a warp may touch only the TMEM lane quarter warp % 4, so a
// strip narrower than 128 columns spreads S k ranges over the quarters instead (S = 4 for 1 unit, 2 for <= 2).
__host__ __device__ inline int umma_split(int units, int k, int step_k) {
  if (units == 1 && k % (4 * step_k) == 0) return 4;
  if (units <= 2 && k % (2 * step_k) == 0) return 2;
  return 1;
}

// Walks a CTA's strips (<= 4 units of 32 columns) and their k steps in the one order every warp role follows.
struct UmmaCursor {
  int unit, unit_end, k, step_k;  // next strip starts at `unit`
  int force_split;                 // 0: umma_split decides per strip; else every strip uses this split
  int units, split, steps, kper;  // current strip: units, k ranges, steps per range, k per range
  int kc;                          // step inside the strip
  int q;                           // steps since the kernel started
  __device__ void init(int cta, int ctas, int total_units, int k_, int step_k_, int force_split_ = 0) {
    force_split = force_split_;
    unit = static_cast<int>(static_cast<int64_t>(cta) * total_units / ctas);
    unit_end = static_cast<int>(static_cast<int64_t>(cta + 1) * total_units / ctas);
    k = k_, step_k = step_k_, q = 0;
  }
  __device__ bool begin_strip() {
    if (unit >= unit_end) return false;
    units = min(force_split ? 4 / force_split : 4, unit_end - unit);
    split = force_split ? force_split : umma_split(units, k, step_k);
    kper = k / split;
    steps = kper / step_k;
    kc = 0;
    return true;
  }
  __device__ bool next_step() {  // false: the strip is finished, the cursor sits on the next one
    ++q;
    if (++kc < steps) return true;
    unit += units;
    return false;
  }
};

}  // namespace xdk
