// Fused rotary embedding + paged K/V cache append for sm_100a: ONE launch rotates Q into q_out,
// rotates K straight into its cache slot and copies V into its cache slot.
//
// Work is cut into "units" of one or two 16-byte vectors.  A rotating unit holds both partners of
// every pair it touches (non-interleaved: the vector at dims [i, i+W) and the one at
// [i + rope_dim/2, ...); interleaved: partners are neighbours inside one vector), so the rotation
// happens in registers.  Each thread issues its payload loads first, then walks the dependent
// index chain (position -> sequence id -> page-table entry) while they are in flight, and finally
// does page-table-translated 128-bit stores.
//
// Bit-exactness: the reference computes a*c - b*s and a*s + b*c as separately rounded FP32
// operations.  __fmul_rn/__fsub_rn/__fadd_rn are never contracted into FMAs, so every K/V byte
// written to the cache and every Q byte equals the PyTorch result.
#include "common.cuh"

namespace xdk {
namespace {

// W elements of T moved as one unit: W == Elem<T>::kPerVec -> one 16-byte vector, W == 1 -> scalar.
template <typename T, int W> struct Chunk {
  float f[W];
  __device__ __forceinline__ void load(const T* p) {
    if constexpr (W == 1) {
      f[0] = Elem<T>::to_f32(*p);
    } else {
      unpack16<T>(ld_stream16(p), f);
    }
  }
  __device__ __forceinline__ void store(T* p) const {
    if constexpr (W == 1) {
      *p = Elem<T>::from_f32(f[0]);
    } else {
      *reinterpret_cast<U4*>(p) = pack16<T>(f);
    }
  }
};

struct RopeShape {
  int q_heads, kv_heads, head_dim, rope_dim;
  int cos_width, page_size;
  int64_t max_pages;
  int64_t q_stride, k_stride, v_stride;  // elements between consecutive tokens of q, k, v
  int hnd;
  PeerOut qout;  // rotated Q: row = token, column = head * head_dim + dim (plus col0), in every destination
};

// Element offset of (page, offset, head, dim 0) in a contiguous cache; identical integers to the
// host helpers nhd_linear_index / hnd_linear_index.
__device__ __forceinline__ int64_t cache_row(const RopeShape& s, int64_t page, int64_t off, int head) {
  return s.hnd ? ((page * s.kv_heads + head) * s.page_size + off) * s.head_dim
               : ((page * s.page_size + off) * s.kv_heads + head) * s.head_dim;
}

template <typename T, int W, bool INTERLEAVED>
__global__ void __launch_bounds__(128)
rope_append_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                   const float* __restrict__ cos, const float* __restrict__ sin,
                   const int64_t* __restrict__ positions, const int64_t* __restrict__ page_table,
                   const int64_t* __restrict__ sequence_ids, T* __restrict__ q_out, T* __restrict__ k_cache,
                   T* __restrict__ v_cache, RopeShape s, int units_rot_head, int units_token) {
  pdl_launch_dependents();
  pdl_wait();  // q, k, v may be the preceding kernel's output; the caches may still be read by it
  const int token = blockIdx.x;
  const int unit = blockIdx.y * 128 + threadIdx.x;
  if (unit >= units_token) return;

  const int vecs = s.head_dim / W;              // W-wide chunks per head
  const int rot_vecs = s.rope_dim / W;          // of which rotated (exact division on this path)
  const int pair_vecs = rot_vecs / 2;           // non-interleaved: chunks per half
  const int rot_heads = s.q_heads + s.kv_heads;  // heads that go through the rotation

  // ---- decode the unit: which tensor/head, which chunk(s), rotate or copy
  int head, first, second = -1;  // chunk indices inside the head (second < 0: single-chunk unit)
  bool rotate = false;
  int kind;  // 0 = Q, 1 = K, 2 = V
  if (unit < rot_heads * units_rot_head) {
    head = unit / units_rot_head;
    const int u = unit - head * units_rot_head;
    kind = head < s.q_heads ? 0 : 1;
    if (kind == 1) head -= s.q_heads;
    if (INTERLEAVED) {
      first = u;
      rotate = u < rot_vecs;
    } else if (u < pair_vecs) {
      first = u;
      second = u + pair_vecs;
      rotate = true;
    } else {
      first = rot_vecs + (u - pair_vecs);
    }
  } else {
    const int u = unit - rot_heads * units_rot_head;
    head = u / vecs;
    first = u - head * vecs;
    kind = 2;
  }

  // ---- payload loads first (independent of every index)
  const T* src = kind == 0 ? q : (kind == 1 ? k : v);
  const int64_t stride = kind == 0 ? s.q_stride : (kind == 1 ? s.k_stride : s.v_stride);
  const int64_t src_row = static_cast<int64_t>(token) * stride + static_cast<int64_t>(head) * s.head_dim;
  Chunk<T, W> a, b;
  a.load(src + src_row + static_cast<int64_t>(first) * W);
  if (second >= 0) b.load(src + src_row + static_cast<int64_t>(second) * W);

  // ---- dependent index chain
  const int64_t pos = __ldg(positions + token);
  int64_t dst_row = static_cast<int64_t>(token) * s.qout.ld + s.qout.col0 + static_cast<int64_t>(head) * s.head_dim;
  T* dst = q_out;
  if (kind != 0) {
    const int64_t seq = __ldg(sequence_ids + token);
    const int64_t logical = pos / s.page_size;
    const int64_t off = pos - logical * s.page_size;
    const int64_t page = __ldg(page_table + seq * s.max_pages + logical);
    dst_row = cache_row(s, page, off, head);
    dst = kind == 1 ? k_cache : v_cache;
  }

  if (rotate) {
    const float* crow = cos + pos * s.cos_width;
    const float* srow = sin + pos * s.cos_width;
    if (INTERLEAVED) {
      // chunk `first` holds pairs (2i, 2i+1) for i in [first*W/2, first*W/2 + W/2)
      const int pair0 = first * (W / 2);
#pragma unroll
      for (int e = 0; e < W / 2; ++e) {
        const float c = __ldg(crow + pair0 + e), sn = __ldg(srow + pair0 + e);
        const float lo = a.f[2 * e], hi = a.f[2 * e + 1];
        a.f[2 * e] = __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, sn));
        a.f[2 * e + 1] = __fadd_rn(__fmul_rn(lo, sn), __fmul_rn(hi, c));
      }
    } else {
      const int pair0 = first * W;
#pragma unroll
      for (int e = 0; e < W; ++e) {
        const float c = __ldg(crow + pair0 + e), sn = __ldg(srow + pair0 + e);
        const float lo = a.f[e], hi = b.f[e];
        a.f[e] = __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, sn));
        b.f[e] = __fadd_rn(__fmul_rn(lo, sn), __fmul_rn(hi, c));
      }
    }
  }
  a.store(dst + dst_row + static_cast<int64_t>(first) * W);
  if (second >= 0) b.store(dst + dst_row + static_cast<int64_t>(second) * W);
  if (kind == 0) {  // the other ranks' copies of the rotated Q
#pragma unroll 1
    for (int p = 1; p < s.qout.world; ++p) {
      T* peer = static_cast<T*>(s.qout.ptr[p]);
      a.store(peer + dst_row + static_cast<int64_t>(first) * W);
      if (second >= 0) b.store(peer + dst_row + static_cast<int64_t>(second) * W);
    }
  }
}

template <typename T, int W, bool INTERLEAVED>
int launch_rope(const void* q, const void* k, const void* v, const float* cos, const float* sin,
                const int64_t* positions, const int64_t* page_table, const int64_t* sequence_ids, void* q_out,
                void* k_cache, void* v_cache, int64_t tokens, const RopeShape& s, cudaStream_t stream) {
  const int vecs = s.head_dim / W, rot_vecs = s.rope_dim / W;
  const int units_rot_head = INTERLEAVED ? vecs : rot_vecs / 2 + (vecs - rot_vecs);
  const int64_t units_token64 =
      static_cast<int64_t>(s.q_heads + s.kv_heads) * units_rot_head + static_cast<int64_t>(s.kv_heads) * vecs;
  if (units_token64 > 65535LL * 128) return XDK_ERR_LIMIT;
  const int units_token = static_cast<int>(units_token64);
  dim3 grid(static_cast<unsigned>(tokens), static_cast<unsigned>((units_token + 127) / 128));
  return launch_dependent(rope_append_kernel<T, W, INTERLEAVED>, grid, dim3(128), 0, stream, static_cast<const T*>(q),
                static_cast<const T*>(k), static_cast<const T*>(v), cos, sin, positions, page_table, sequence_ids,
                static_cast<T*>(q_out), static_cast<T*>(k_cache), static_cast<T*>(v_cache), s, units_rot_head,
                units_token);
}

// Scalar interleaved path: one thread per (head, pair) or per copied element.
template <typename T>
__global__ void __launch_bounds__(128)
rope_append_scalar_interleaved_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                      const float* __restrict__ cos, const float* __restrict__ sin,
                                      const int64_t* __restrict__ positions, const int64_t* __restrict__ page_table,
                                      const int64_t* __restrict__ sequence_ids, T* __restrict__ q_out,
                                      T* __restrict__ k_cache, T* __restrict__ v_cache, RopeShape s,
                                      int units_rot_head, int units_token) {
  pdl_launch_dependents();
  pdl_wait();  // q, k, v may be the preceding kernel's output; the caches may still be read by it
  const int token = blockIdx.x;
  const int unit = blockIdx.y * 128 + threadIdx.x;
  if (unit >= units_token) return;
  const int pairs = s.rope_dim / 2;
  const int rot_heads = s.q_heads + s.kv_heads;
  int head, kind, d0, d1 = -1;
  if (unit < rot_heads * units_rot_head) {
    head = unit / units_rot_head;
    const int u = unit - head * units_rot_head;
    kind = head < s.q_heads ? 0 : 1;
    if (kind == 1) head -= s.q_heads;
    if (u < pairs) {
      d0 = 2 * u;
      d1 = 2 * u + 1;
    } else {
      d0 = s.rope_dim + (u - pairs);
    }
  } else {
    const int u = unit - rot_heads * units_rot_head;
    head = u / s.head_dim;
    d0 = u - head * s.head_dim;
    kind = 2;
  }
  const T* src = kind == 0 ? q : (kind == 1 ? k : v);
  const int64_t stride = kind == 0 ? s.q_stride : (kind == 1 ? s.k_stride : s.v_stride);
  const int64_t src_row = static_cast<int64_t>(token) * stride + static_cast<int64_t>(head) * s.head_dim;
  float lo = Elem<T>::to_f32(src[src_row + d0]);
  float hi = d1 >= 0 ? Elem<T>::to_f32(src[src_row + d1]) : 0.0f;
  const int64_t pos = __ldg(positions + token);
  int64_t dst_row = static_cast<int64_t>(token) * s.qout.ld + s.qout.col0 + static_cast<int64_t>(head) * s.head_dim;
  T* dst = q_out;
  if (kind != 0) {
    const int64_t seq = __ldg(sequence_ids + token);
    const int64_t logical = pos / s.page_size;
    const int64_t off = pos - logical * s.page_size;
    const int64_t page = __ldg(page_table + seq * s.max_pages + logical);
    dst_row = cache_row(s, page, off, head);
    dst = kind == 1 ? k_cache : v_cache;
  }
  if (d1 >= 0) {
    const float c = __ldg(cos + pos * s.cos_width + d0 / 2), sn = __ldg(sin + pos * s.cos_width + d0 / 2);
    const float new_lo = __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, sn));
    const float new_hi = __fadd_rn(__fmul_rn(lo, sn), __fmul_rn(hi, c));
    dst[dst_row + d0] = Elem<T>::from_f32(new_lo);
    dst[dst_row + d1] = Elem<T>::from_f32(new_hi);
    if (kind == 0)
      for (int p = 1; p < s.qout.world; ++p) {
        static_cast<T*>(s.qout.ptr[p])[dst_row + d0] = Elem<T>::from_f32(new_lo);
        static_cast<T*>(s.qout.ptr[p])[dst_row + d1] = Elem<T>::from_f32(new_hi);
      }
  } else {
    dst[dst_row + d0] = Elem<T>::from_f32(lo);
    if (kind == 0)
      for (int p = 1; p < s.qout.world; ++p) static_cast<T*>(s.qout.ptr[p])[dst_row + d0] = Elem<T>::from_f32(lo);
  }
}

template <typename T>
int dispatch_all(const void* q, const void* k, const void* v, const float* cos, const float* sin,
                 const int64_t* positions, const int64_t* page_table, const int64_t* sequence_ids, void* q_out,
                 void* k_cache, void* v_cache, int64_t tokens, const RopeShape& s, bool interleaved,
                 cudaStream_t stream) {
  constexpr int E = Elem<T>::kPerVec;
  bool aligned = aligned16(q) && aligned16(k) && aligned16(v) && aligned16(k_cache) && aligned16(v_cache) &&
                 s.qout.ld % E == 0 && s.qout.col0 % E == 0;
  for (int p = 0; p < s.qout.world; ++p) aligned = aligned && aligned16(s.qout.ptr[p]);
  // Vector path: whole 16-byte chunks, and rotation partners that fall on chunk boundaries.
  const bool vec = aligned && s.head_dim % E == 0 && s.q_stride % E == 0 && s.k_stride % E == 0 &&
                   s.v_stride % E == 0 && (interleaved ? s.rope_dim % E == 0 : (s.rope_dim / 2) % E == 0);
#define XDK_ROPE(WW, IL)                                                                                          \
  return launch_rope<T, WW, IL>(q, k, v, cos, sin, positions, page_table, sequence_ids, q_out, k_cache, v_cache, \
                                tokens, s, stream)
  if (vec && interleaved) XDK_ROPE(E, true);
  if (vec) XDK_ROPE(E, false);
  // Odd head sizes or unaligned views: element-wise units.
  if (!interleaved) XDK_ROPE(1, false);
#undef XDK_ROPE
  const int units_rot_head = s.rope_dim / 2 + (s.head_dim - s.rope_dim);
  const int64_t units_token64 =
      static_cast<int64_t>(s.q_heads + s.kv_heads) * units_rot_head + static_cast<int64_t>(s.kv_heads) * s.head_dim;
  if (units_token64 > 65535LL * 128) return XDK_ERR_LIMIT;
  const int units_token = static_cast<int>(units_token64);
  dim3 grid(static_cast<unsigned>(tokens), static_cast<unsigned>((units_token + 127) / 128));
  return launch_dependent(rope_append_scalar_interleaved_kernel<T>, grid, dim3(128), 0, stream, static_cast<const T*>(q),
                static_cast<const T*>(k), static_cast<const T*>(v), cos, sin, positions, page_table, sequence_ids,
                static_cast<T*>(q_out), static_cast<T*>(k_cache), static_cast<T*>(v_cache), s, units_rot_head,
                units_token);
}

}  // namespace
}  // namespace xdk

extern "C" int xdk_rope_kv_append(const void* q, const void* k, const void* v, const float* cos, const float* sin,
                                  const int64_t* positions, const int64_t* page_table, const int64_t* sequence_ids,
                                  void* q_out, void* k_cache, void* v_cache, int64_t tokens, int64_t q_heads,
                                  int64_t kv_heads, int64_t head_dim, int64_t cos_width, int64_t max_pages_per_seq,
                                  int64_t page_size, int64_t rope_dim, int64_t q_token_stride, int64_t k_token_stride,
                                  int64_t v_token_stride, int interleaved, int cache_is_hnd, int dtype,
                                  void* stream) {
  return xdk_rope_kv_append_v2(q, k, v, cos, sin, positions, page_table, sequence_ids, q_out, k_cache, v_cache, tokens,
                               q_heads, kv_heads, head_dim, cos_width, max_pages_per_seq, page_size, rope_dim,
                               q_token_stride, k_token_stride, v_token_stride, interleaved, cache_is_hnd, dtype, 0u, stream);
}

extern "C" int xdk_rope_kv_append_v2(const void* q, const void* k, const void* v, const float* cos, const float* sin,
                                     const int64_t* positions, const int64_t* page_table, const int64_t* sequence_ids,
                                     void* q_out, void* k_cache, void* v_cache, int64_t tokens, int64_t q_heads,
                                     int64_t kv_heads, int64_t head_dim, int64_t cos_width, int64_t max_pages_per_seq,
                                     int64_t page_size, int64_t rope_dim, int64_t q_token_stride, int64_t k_token_stride,
                                     int64_t v_token_stride, int interleaved, int cache_is_hnd, int dtype,
                                     unsigned flags, void* stream) {
  if (!q_out || q_heads <= 0 || head_dim <= 0) return XDK_ERR_ARG;
  xdk_peer_out one = {};
  one.ptr[0] = q_out, one.world = 1, one.ld = q_heads * head_dim, one.col0 = 0;
  return xdk_rope_kv_append_peer(q, k, v, cos, sin, positions, page_table, sequence_ids, &one, k_cache, v_cache, tokens,
                                 q_heads, kv_heads, head_dim, cos_width, max_pages_per_seq, page_size, rope_dim,
                                 q_token_stride, k_token_stride, v_token_stride, interleaved, cache_is_hnd, dtype, flags,
                                 stream);
}

extern "C" int xdk_rope_kv_append_peer(const void* q, const void* k, const void* v, const float* cos, const float* sin,
                                       const int64_t* positions, const int64_t* page_table, const int64_t* sequence_ids,
                                       const xdk_peer_out* q_dst, void* k_cache, void* v_cache, int64_t tokens,
                                       int64_t q_heads, int64_t kv_heads, int64_t head_dim, int64_t cos_width,
                                       int64_t max_pages_per_seq, int64_t page_size, int64_t rope_dim,
                                       int64_t q_token_stride, int64_t k_token_stride, int64_t v_token_stride,
                                       int interleaved, int cache_is_hnd, int dtype, unsigned flags, void* stream) {
  if (flags & ~XDK_DEPENDENT_LAUNCH) return XDK_ERR_ARG;
  xdk::CallFlagsScope scope(flags);
  xdk::PeerOut qout;
  if (int st = xdk::make_out(q_dst, nullptr, 1, &qout)) return st;
  if (q_heads > 0 && head_dim > 0 && qout.ld < qout.col0 + q_heads * head_dim) return XDK_ERR_ARG;
  void* q_out = qout.ptr[0];
  if (!q || !k || !v || !cos || !sin || !positions || !page_table || !sequence_ids || !q_out || !k_cache || !v_cache)
    return XDK_ERR_ARG;
  if (tokens <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || page_size <= 0 || max_pages_per_seq <= 0)
    return XDK_ERR_ARG;
  if (q_heads % kv_heads != 0) return XDK_ERR_ARG;
  if (rope_dim <= 0 || rope_dim % 2 != 0 || rope_dim > head_dim || cos_width < rope_dim / 2) return XDK_ERR_ARG;
  if (q_token_stride < q_heads * head_dim || k_token_stride < kv_heads * head_dim ||
      v_token_stride < kv_heads * head_dim)
    return XDK_ERR_ARG;
  const int64_t int_max = 2147483647LL;
  if (tokens > int_max || q_heads > 65535 || kv_heads > 65535 || head_dim > 65536 || cos_width > int_max ||
      page_size > int_max)
    return XDK_ERR_LIMIT;
  if (int st = xdk::require_sm100()) return st;
  xdk::RopeShape s;
  s.q_heads = static_cast<int>(q_heads);
  s.kv_heads = static_cast<int>(kv_heads);
  s.head_dim = static_cast<int>(head_dim);
  s.rope_dim = static_cast<int>(rope_dim);
  s.cos_width = static_cast<int>(cos_width);
  s.page_size = static_cast<int>(page_size);
  s.max_pages = max_pages_per_seq;
  s.q_stride = q_token_stride, s.k_stride = k_token_stride, s.v_stride = v_token_stride;
  s.hnd = cache_is_hnd ? 1 : 0;
  s.qout = qout;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool il = interleaved != 0;
  switch (dtype) {
    case XDK_F32:
      return xdk::dispatch_all<float>(q, k, v, cos, sin, positions, page_table, sequence_ids, q_out, k_cache, v_cache,
                                      tokens, s, il, st);
    case XDK_BF16:
      return xdk::dispatch_all<__nv_bfloat16>(q, k, v, cos, sin, positions, page_table, sequence_ids, q_out, k_cache,
                                              v_cache, tokens, s, il, st);
    case XDK_F16:
      return xdk::dispatch_all<__half>(q, k, v, cos, sin, positions, page_table, sequence_ids, q_out, k_cache,
                                       v_cache, tokens, s, il, st);
    default:
      return XDK_ERR_ARG;
  }
}
