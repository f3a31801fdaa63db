// Peer-mapped output buffers and the flag barrier of the multi-GPU path (one process per GPU, one node).
//
// Every rank allocates an arena of the same size with cudaMalloc, exports it as a CUDA IPC handle, and maps
// the arenas of the other ranks (the handles travel through the host-side process group).  A kernel whose
// output is column-sharded then stores its tile straight into the same offset of every rank's arena (PeerOut,
// common.cuh) -- plain st.global over NVLink, no multicast, no TMA.  Readers are ordered after writers by
// peer_barrier_kernel: launched on every rank after the producing kernels, it publishes this rank's epoch to
// every peer with a system-scope release store and waits, for a bounded time, until every peer has published
// the same epoch.  A wait that runs out sets a bit in the fault word and the kernel returns; nothing spins
// for ever.  The epoch lives on the device and advances by itself, so the barrier can sit in a CUDA graph
// that is replayed.
#include <string.h>

#include "common.cuh"

namespace xdk {
namespace {

__device__ unsigned int g_peer_fault;  // bit p: the wait on peer p gave up at some point

// Arena layout (host and device agree): the first kFlagBytes hold, per barrier site s < kSites,
//   uint64 arrived[s][XDK_MAX_PEERS]   written by the peers (slot = writer's rank)
//   uint64 epoch[s]                    this rank's own count of barriers passed at the site
constexpr int kSites = 64;
struct FlagBlock {
  unsigned long long arrived[kSites][XDK_MAX_PEERS];
  unsigned long long epoch[kSites];
};
static_assert(sizeof(FlagBlock) <= XDK_PEER_FLAG_BYTES, "flag block must fit the reserved head of the arena");

struct BarrierArgs {
  FlagBlock* flags[XDK_MAX_PEERS];  // flags[p]: the flag block of rank p (flags[rank] is local)
  int rank, world, site;
  unsigned long long budget_ns;
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(BarrierArgs a) {
  pdl_launch_dependents();
  pdl_wait();  // the producing kernels of this stream have completed: their peer stores are performed
  const int p = threadIdx.x;
  FlagBlock* mine = a.flags[a.rank];
  unsigned long long epoch = 0;
  if (p == 0) {
    epoch = mine->epoch[a.site] + 1;
    mine->epoch[a.site] = epoch;
  }
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  if (p < a.world) {
    __threadfence_system();
    // publish: slot `rank` of the site on peer p (on ourselves too: the wait below is then uniform)
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(&a.flags[p]->arrived[a.site][a.rank]), "l"(epoch) : "memory");
    const unsigned long long* slot = &mine->arrived[a.site][p];
    const uint64_t t0 = global_timer_ns();
    for (;;) {
      unsigned long long seen;
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(slot) : "memory");
      if (seen >= epoch) break;
      if (global_timer_ns() - t0 > a.budget_ns) {
        atomicOr(&g_peer_fault, 1u << p);
        break;
      }
      __nanosleep(100);
    }
  }
}

}  // namespace

unsigned peer_fault_word() {
  unsigned v = 0;
  if (cudaMemcpyFromSymbol(&v, g_peer_fault, sizeof(v)) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0x80000000u;
  }
  return v;
}

int make_out(const xdk_peer_out* peers, void* fallback, int64_t ld, PeerOut* out) {
  if (!peers) {
    if (!fallback) return XDK_ERR_ARG;
    *out = single_out(fallback, ld);
    return XDK_OK;
  }
  if (peers->world < 1 || peers->world > XDK_MAX_PEERS || peers->ld < 1 || peers->col0 < 0) return XDK_ERR_ARG;
  *out = PeerOut{};
  for (int p = 0; p < peers->world; ++p) {
    if (!peers->ptr[p]) return XDK_ERR_ARG;
    out->ptr[p] = peers->ptr[p];
  }
  out->world = peers->world;
  out->ld = peers->ld;
  out->col0 = peers->col0;
  return XDK_OK;
}

}  // namespace xdk

extern "C" {

int xdk_peer_alloc(size_t bytes, void** ptr) {
  if (!ptr || bytes < XDK_PEER_FLAG_BYTES) return XDK_ERR_ARG;
  void* p = nullptr;
  cudaError_t err = cudaMalloc(&p, bytes);
  if (err != cudaSuccess) return xdk::note_launch(err);
  err = cudaMemset(p, 0, bytes);
  if (err != cudaSuccess) {
    (void)cudaFree(p);
    return xdk::note_launch(err);
  }
  *ptr = p;
  return XDK_OK;
}

int xdk_peer_free(void* ptr) { return ptr ? xdk::note_launch(cudaFree(ptr)) : XDK_OK; }

int xdk_peer_export(void* ptr, void* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  if (!ptr || !handle64) return XDK_ERR_ARG;
  return xdk::note_launch(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), ptr));
}

int xdk_peer_open(const void* handle64, void** ptr) {
  if (!handle64 || !ptr) return XDK_ERR_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return xdk::note_launch(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}

int xdk_peer_close(void* ptr) { return ptr ? xdk::note_launch(cudaIpcCloseMemHandle(ptr)) : XDK_OK; }

int xdk_peer_barrier(void* const* arenas, int rank, int world, int site, unsigned timeout_us, unsigned flags, void* stream) {
  using namespace xdk;
  if (!arenas || world < 1 || world > XDK_MAX_PEERS || rank < 0 || rank >= world || site < 0 || site >= kSites)
    return XDK_ERR_ARG;
  if (flags & ~XDK_DEPENDENT_LAUNCH) return XDK_ERR_ARG;
  if (int st = require_sm100()) return st;
  BarrierArgs a = {};
  for (int p = 0; p < world; ++p) {
    if (!arenas[p]) return XDK_ERR_ARG;
    a.flags[p] = static_cast<FlagBlock*>(arenas[p]);
  }
  a.rank = rank, a.world = world, a.site = site;
  a.budget_ns = static_cast<unsigned long long>(timeout_us ? timeout_us : 1000000u) * 1000ull;
  return launch_opts(peer_barrier_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), 1u,
                     (flags & XDK_DEPENDENT_LAUNCH) != 0, a);
}

}  // extern "C"
