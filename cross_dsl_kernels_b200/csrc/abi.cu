// Status codes, error text and the device gate of the C ABI.
#include "common.cuh"

namespace xdk {

static thread_local int g_last_cuda_error = 0;
static thread_local unsigned g_call_flags = 0;

unsigned call_flags() { return g_call_flags; }
void set_call_flags(unsigned flags) { g_call_flags = flags; }

int note_launch(cudaError_t err) {
  if (err == cudaSuccess) return XDK_OK;
  g_last_cuda_error = static_cast<int>(err);
  (void)cudaGetLastError();  // clear the sticky-free launch error so later calls start clean
  return XDK_ERR_LAUNCH;
}

int require_sm100() {
  static int verdict[64];  // 0 = unknown, 1 = ok, 2 = wrong architecture
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) {
    (void)cudaGetLastError();
    return XDK_ERR_ARCH;
  }
  if (dev < 64 && verdict[dev]) return verdict[dev] == 1 ? XDK_OK : XDK_ERR_ARCH;
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return XDK_ERR_ARCH;
  }
  if (dev < 64) verdict[dev] = major == 10 ? 1 : 2;
  return major == 10 ? XDK_OK : XDK_ERR_ARCH;
}

bool encode_tiled(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base, const cuuint64_t* dims,
                  const cuuint64_t* strides_bytes, const cuuint32_t* box, bool swizzle128) {
  using Encode = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Encode encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) {
      (void)cudaGetLastError();
      return false;
    }
    encode = reinterpret_cast<Encode>(fn);
  }
  const cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
  if (rank < 1 || rank > 5) return false;
  return encode(map, type, static_cast<cuuint32_t>(rank), const_cast<void*>(base), dims, strides_bytes, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool encode_tiled_2d(CUtensorMap* map, CUtensorMapDataType type, const void* base, const cuuint64_t* dims,
                     const cuuint64_t* strides_bytes, const cuuint32_t* box, bool swizzle128) {
  return encode_tiled(map, type, 2, base, dims, strides_bytes, box, swizzle128);
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

namespace {
__global__ void noop_kernel() {
  pdl_launch_dependents();
  pdl_wait();
}
}  // namespace

}  // namespace xdk

extern "C" {

int xdk_noop(unsigned flags, void* stream) {
  if (flags & ~XDK_DEPENDENT_LAUNCH) return XDK_ERR_ARG;
  if (int st = xdk::require_sm100()) return st;
  return xdk::launch_opts(xdk::noop_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), 1u,
                          (flags & XDK_DEPENDENT_LAUNCH) != 0);
}

const char* xdk_strerror(int status) {
  switch (status) {
    case XDK_OK: return "ok";
    case XDK_ERR_ARG: return "invalid argument (size, enum or null pointer)";
    case XDK_ERR_ARCH: return "current CUDA device is not compute capability 10.x (B200, sm_100a)";
    case XDK_ERR_LAUNCH: return "CUDA runtime refused the kernel launch (see xdk_last_cuda_error)";
    case XDK_ERR_LIMIT: return "size beyond what this build supports";
    default: return "unknown xdk status";
  }
}

int xdk_abi_version(void) { return XDK_ABI_VERSION; }

int xdk_last_cuda_error(void) { return xdk::g_last_cuda_error; }

unsigned xdk_fault_flags(void) {
  const unsigned words[3] = {xdk::gemv_fault_word(), xdk::w4a16_fault_word(), xdk::gemv_tc_fault_word()};
  unsigned out = 0;
  for (int i = 0; i < 3; ++i) {
    if (words[i] & 0x80000000u) out |= 0x80000000u;  // the word could not be read: never report "healthy"
    out |= (words[i] & 0x7fu) << (8 * i);
  }
  return out;
}

unsigned xdk_peer_fault_flags(void) { return xdk::peer_fault_word(); }

int xdk_device_supported(int device) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    (void)cudaGetLastError();
    return XDK_ERR_ARCH;
  }
  if (device < 0 || device >= count) return XDK_ERR_ARG;
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
    (void)cudaGetLastError();
    return XDK_ERR_ARCH;
  }
  return major == 10 ? XDK_OK : XDK_ERR_ARCH;
}

}  // extern "C"
