// SwiGLU on the output of the fused up+gate projection:  out[m][j] = silu(gate[m][j]) * up[m][j].
//
// The up+gate projection of the decode layer writes [rows, 2 * width]: columns [0, width) are "up", columns
// [width, 2 * width) are "gate" (the order of the rows of the fused weight).  The op after it in a Llama-style MLP
// multiplies up by silu(gate) = gate / (1 + exp(-gate)) and hands [rows, width] to the down projection.  FP32
// arithmetic on 16-byte vectors, one rounding to the storage type.  Not part of upstream (its chain stops at the
// projection); the expectation is this library's own FP32 restatement of the formula.
#include "common.cuh"

namespace xdk {
namespace {

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_kernel(const T* __restrict__ upgate, const PeerOut out, int64_t rows, int64_t width_vecs, int64_t in_ld) {
  constexpr int E = Elem<T>::kPerVec;
  pdl_launch_dependents();
  pdl_wait();  // upgate is the preceding kernel's output
  const int64_t total = rows * width_vecs;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t r = i / width_vecs, v = i - r * width_vecs;
    const T* row = upgate + r * in_ld;
    float up[E], gate[E], res[E];
    unpack16<T>(ld_stream16(row + v * E), up);
    unpack16<T>(ld_stream16(row + (width_vecs + v) * E), gate);
#pragma unroll
    for (int e = 0; e < E; ++e) res[e] = __fmul_rn(__fdiv_rn(gate[e], __fadd_rn(1.0f, expf(-gate[e]))), up[e]);
    const U4 packed = pack16<T>(res);
    const int64_t at = r * out.ld + out.col0 + v * E;
#pragma unroll 1
    for (int p = 0; p < out.world; ++p) st_stream16(static_cast<T*>(out.ptr[p]) + at, packed);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_scalar_kernel(const T* __restrict__ upgate, const PeerOut out, int64_t rows, int64_t width, int64_t in_ld) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = rows * width;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t r = i / width, c = i - r * width;
    const float up = Elem<T>::to_f32(upgate[r * in_ld + c]), gate = Elem<T>::to_f32(upgate[r * in_ld + width + c]);
    peer_store(out, r, c, Elem<T>::from_f32(__fmul_rn(__fdiv_rn(gate, __fadd_rn(1.0f, expf(-gate))), up)));
  }
}

template <typename T>
int dispatch(const void* upgate, const PeerOut& out, int64_t rows, int64_t width, int64_t in_ld, cudaStream_t s) {
  constexpr int E = Elem<T>::kPerVec;
  bool vec = width % E == 0 && in_ld % E == 0 && out.ld % E == 0 && out.col0 % E == 0 && aligned16(upgate);
  for (int p = 0; p < out.world; ++p) vec = vec && aligned16(out.ptr[p]);
  const int64_t items = vec ? rows * (width / E) : rows * width;
  int64_t blocks = (items + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  if (vec)
    return launch_dependent(swiglu_kernel<T>, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, s, static_cast<const T*>(upgate),
                            out, rows, width / E, in_ld);
  return launch_dependent(swiglu_scalar_kernel<T>, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, s,
                          static_cast<const T*>(upgate), out, rows, width, in_ld);
}

}  // namespace
}  // namespace xdk

extern "C" int xdk_swiglu(const void* upgate, void* out, int64_t rows, int64_t width, int64_t in_ld, int64_t out_ld, int dtype,
                          unsigned flags, void* stream) {
  if (!out || out_ld < width) return XDK_ERR_ARG;
  xdk_peer_out one = {};
  one.ptr[0] = out, one.world = 1, one.ld = out_ld, one.col0 = 0;
  return xdk_swiglu_peer(upgate, &one, rows, width, in_ld, dtype, flags, stream);
}

extern "C" int xdk_swiglu_peer(const void* upgate, const xdk_peer_out* out_dst, int64_t rows, int64_t width, int64_t in_ld, int dtype,
                               unsigned flags, void* stream) {
  if (flags & ~XDK_DEPENDENT_LAUNCH) return XDK_ERR_ARG;
  xdk::CallFlagsScope scope(flags);
  xdk::PeerOut out;
  if (int st = xdk::make_out(out_dst, nullptr, 1, &out)) return st;
  if (!upgate || rows < 1 || width < 1 || in_ld < 2 * width || out.ld < out.col0 + width) return XDK_ERR_ARG;
  if (rows > (1LL << 40) / width) return XDK_ERR_LIMIT;
  if (int st = xdk::require_sm100()) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case XDK_F32: return xdk::dispatch<float>(upgate, out, rows, width, in_ld, s);
    case XDK_BF16: return xdk::dispatch<__nv_bfloat16>(upgate, out, rows, width, in_ld, s);
    case XDK_F16: return xdk::dispatch<__half>(upgate, out, rows, width, in_ld, s);
    default: return XDK_ERR_ARG;
  }
}
