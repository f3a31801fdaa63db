// Shared device/host helpers for the sm_100a decode kernels.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/xdk_b200.h"

namespace xdk {

// ---- host side -------------------------------------------------------------------------------

// Records the runtime's error for xdk_last_cuda_error() and maps it to a status.
int note_launch(cudaError_t err);
// XDK_OK when the device current to this thread is compute capability 10.x (cached per device).
int require_sm100();

// Encodes a tiled TMA tensor map of `rank` dimensions (dims/box: rank entries, innermost first;
// strides_bytes: rank - 1 entries, for dims 1 ..).  cuTensorMapEncodeTiled is fetched from the driver
// through the runtime, so the library has no link-time dependency on libcuda.  swizzle128: 128-byte
// swizzle (inner box must be 128 bytes).  encode_tiled_2d is the rank-2 shorthand.
bool encode_tiled(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base, const cuuint64_t* dims,
                  const cuuint64_t* strides_bytes, const cuuint32_t* box, bool swizzle128);
bool encode_tiled_2d(CUtensorMap* map, CUtensorMapDataType type, const void* base, const cuuint64_t* dims,
                     const cuuint64_t* strides_bytes, const cuuint32_t* box, bool swizzle128);
int sm_count();  // SMs of the current device (cached per device)
// Fault words of the kernels with bounded waits (current device; synchronises).  0 = no wait ever gave up.
unsigned gemv_fault_word();
unsigned gemv_tc_fault_word();
unsigned w4a16_fault_word();

// tcgen05 FP32 projection (gemv_tc.cu): whether it takes the shape, and its launch
bool gemv_tc_eligible(const float* x, const float* w, int64_t m, int64_t k, int64_t n, bool nk);
int gemv_tc_plan(int64_t m, int64_t k, int64_t n, bool nk, int32_t out[5]);  // {CTAs, lane-quarter K split, ring depth, smem bytes, units}; returns the cluster size, 0 = declined

// Flags of the *_v2 entry point that is executing on this host thread (0 outside one).
unsigned call_flags();
void set_call_flags(unsigned flags);
struct CallFlagsScope {  // sets the flags for the duration of one entry point
  explicit CallFlagsScope(unsigned flags) { set_call_flags(flags); }
  ~CallFlagsScope() { set_call_flags(0u); }
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename... Args>
inline int launch_opts(void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       unsigned cluster_y, bool dependent, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n_attr = 0;
  if (cluster_y > 1) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 1;
    attr[n_attr].val.clusterDim.y = cluster_y;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  if (dependent) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  return note_launch(cudaLaunchKernelEx(&cfg, kernel, args...));
}
template <typename... Args>
inline int launch(void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                  unsigned cluster_y, Args... args) {
  return launch_opts(kernel, grid, block, smem, stream, cluster_y, false, args...);
}
// For kernels that execute pdl_wait() before they touch anything the preceding kernel of the stream wrote:
// launched as a programmatic dependent of that kernel when the executing entry point was given
// XDK_DEPENDENT_LAUNCH, so their scheduling and set-up overlap its tail.
template <typename... Args>
inline int launch_dependent(void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            Args... args) {
  return launch_opts(kernel, grid, block, smem, stream, 1u, (call_flags() & XDK_DEPENDENT_LAUNCH) != 0, args...);
}

// ---- where a kernel's output matrix goes --------------------------------------------------------
// Either the caller's own buffer (world == 1), or the same place in EVERY rank's full-width buffer: rank r of a
// column-sharded projection owns columns [col0, col0 + n) of a [rows, ld] matrix and its epilogue stores each
// value into all `world` copies with ordinary global stores (peer-mapped memory over NVLink).  No collective
// and no re-layout kernel follows; one flag barrier (peer.cu) per exchange point orders readers after writers.
struct PeerOut {
  void* ptr[XDK_MAX_PEERS];
  int world;
  int64_t ld;    // elements between consecutive rows at the destination
  int64_t col0;  // first destination column of this call's output columns
};
inline PeerOut single_out(void* y, int64_t ld) {
  PeerOut o = {};
  o.ptr[0] = y;
  o.world = 1;
  o.ld = ld;
  o.col0 = 0;
  return o;
}
// Copies and checks the caller's descriptor (NULL: `fallback` / `ld` as the only destination).
int make_out(const xdk_peer_out* peers, void* fallback, int64_t ld, PeerOut* out);
unsigned peer_fault_word();
int launch_gemv_tc(const float* x, const float* w, const float* bias, const PeerOut& y, int m, int k, int n, bool nk,
                   cudaStream_t stream);

// ---- device side -----------------------------------------------------------------------------

struct alignas(16) U4 {
  uint32_t x, y, z, w;
};

// 128-bit streaming load: read-only path, do not keep the line in L1 (each byte is used once).
__device__ __forceinline__ U4 ld_stream16(const void* p) {
  U4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// 128-bit load through the read-only cache for data every CTA re-reads (weights of a norm, tables).
__device__ __forceinline__ U4 ld_cached16(const void* p) {
  const uint4 t = __ldg(reinterpret_cast<const uint4*>(p));
  return U4{t.x, t.y, t.z, t.w};
}
__device__ __forceinline__ float4 ld_stream_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_stream_f1(const float* p) {
  float v;
  asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
// 128-bit streaming store (evict-first: the line is not read again by this kernel).
__device__ __forceinline__ void st_stream16(void* p, const U4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Programmatic dependent launch.  pdl_wait: returns once every kernel this one depends on has completed and its
// writes are visible (at once when the launch was an ordinary one).  pdl_launch_dependents: the next kernel of the
// stream, if it was launched as a programmatic dependent, may be scheduled from now on.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename T>
__device__ __forceinline__ void peer_store(const PeerOut& o, int64_t row, int64_t col, T v) {
  const int64_t at = row * o.ld + o.col0 + col;
#pragma unroll 1
  for (int p = 0; p < o.world; ++p) static_cast<T*>(o.ptr[p])[at] = v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
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

// Element <-> float conversions used by the kernels that are generic over storage type.
template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int kPerVec = 4;
  __device__ static __forceinline__ float to_f32(float v) { return v; }
  __device__ static __forceinline__ float from_f32(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int kPerVec = 8;
  __device__ static __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<__half> {
  static constexpr int kPerVec = 8;
  __device__ static __forceinline__ float to_f32(__half v) { return __half2float(v); }
  __device__ static __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};

// Unpack a 16-byte vector of T into floats and back (round-to-nearest-even on the way out).
template <typename T>
__device__ __forceinline__ void unpack16(const U4& v, float (&out)[Elem<T>::kPerVec]) {
  const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int i = 0; i < Elem<T>::kPerVec; ++i) out[i] = Elem<T>::to_f32(e[i]);
}
template <typename T>
__device__ __forceinline__ U4 pack16(const float (&in)[Elem<T>::kPerVec]) {
  U4 v;
  T* e = reinterpret_cast<T*>(&v);
#pragma unroll
  for (int i = 0; i < Elem<T>::kPerVec; ++i) e[i] = Elem<T>::from_f32(in[i]);
  return v;
}

// ---- mbarrier + bulk async copy (global -> this CTA's shared memory) ------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: returns false if the phase did not complete within `budget_ns` of wall time
// (default 20 ms, far beyond any legitimate wait inside these microsecond-scale kernels), so a
// lost copy or a protocol bug can never hang the GPU; callers then skip the work and raise a flag.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, uint64_t budget_ns = 20000000ull) {
  const uint32_t addr = smem_u32(bar);
  uint64_t t0 = 0;
  for (unsigned i = 0;; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
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
// The same bounded wait for roles that mostly wait: every probe lets the hardware park the thread for up to
// `park_ns` (it resumes as soon as the phase completes), so a waiting warp does not take issue slots from the
// warps that compute.
__device__ __forceinline__ bool mbar_wait_parked(uint64_t* bar, unsigned parity, unsigned park_ns = 1000u,
                                                 uint64_t budget_ns = 20000000ull) {
  const uint32_t addr = smem_u32(bar);
  uint64_t t0 = 0;
  for (unsigned i = 0;; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity), "r"(park_ns)
        : "memory");
    if (done) return true;
    if ((i & 3u) == 3u) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_ns) return false;
    }
  }
}
// 1-D bulk copy global -> this CTA's shared memory; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, unsigned bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

}  // namespace xdk
