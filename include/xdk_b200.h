/*
 * xdk_b200.h -- C ABI of the B200 (sm_100a) decode kernels.
 *
 * One shared library, libxdk_b200.so, replaces the four pybind11/ATen modules
 * that upstream (AmanPandey28/cross_dsl_kernels) JIT-builds from
 * csrc/{rmsnorm,gemv,rope_kv,w4a16}.  Every entry point
 *   - takes plain device pointers the caller owns, sizes, and a CUDA stream
 *     (a cudaStream_t passed as void*; NULL is the legacy default stream),
 *   - launches asynchronously on that stream, never synchronises, never
 *     allocates, keeps no state between calls, and may be stream-captured,
 *   - validates sizes and pointers only (tensor-level checks -- dtype, rank,
 *     contiguity, aliasing -- belong to the binding above it),
 *   - returns XDK_OK or a negative xdk_status; it never throws.
 * Paths below are upstream's, relative to its repository root.
 */
#ifndef XDK_B200_H_
#define XDK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XDK_ABI_VERSION 2

#if defined(__GNUC__)
#define XDK_API __attribute__((visibility("default")))
#else
#define XDK_API
#endif

typedef enum xdk_status {
  XDK_OK = 0,
  XDK_ERR_ARG = -1,     /* a size, enum or NULL pointer is not acceptable          */
  XDK_ERR_ARCH = -2,    /* the current device is not compute capability 10.x       */
  XDK_ERR_LAUNCH = -3,  /* the CUDA runtime refused the launch; see xdk_last_cuda_error */
  XDK_ERR_LIMIT = -4    /* a size exceeds what this build supports (stated per call) */
} xdk_status;

/* Storage type of activations for the ops that take more than one. */
typedef enum xdk_dtype {
  XDK_F32 = 0,
  XDK_BF16 = 1,
  XDK_F16 = 2 /* extension: upstream's CUDA kernels take FP32/BF16 only */
} xdk_dtype;

/*
 * Flags of the *_v2 entry points (ABI version 2).  Every *_v2 function takes the arguments of its
 * version-1 namesake plus `unsigned flags` before the stream; the version-1 functions stay and behave
 * as before.
 *   XDK_STRICT_FP32       (xdk_gemv_f32_v2 only) every product and sum is an FP32 FMA on the CUDA cores;
 *                         without it a large 4 < M <= 16 projection may run on the tensor cores as
 *                         split-TF32 products (inside the projection's 1e-5 gate, not bit-identical).
 *                         The choice of arithmetic never depends on whether scratch was passed.
 *   XDK_DEPENDENT_LAUNCH  the kernel is launched as a programmatic dependent of the preceding kernel
 *                         of the stream: it is scheduled while that kernel drains, and waits for that
 *                         kernel's completion on the device before it reads an activation or index
 *                         operand or writes any output.  The caller promises that the CONSTANT
 *                         operands of the call -- projection weights, packed codes, scales, bias,
 *                         norm weight, cos/sin tables -- were not written by the preceding kernel;
 *                         the W4A16 tensor-core kernel starts fetching them before that wait.
 *                         Works eagerly and under stream capture.
 */
#define XDK_STRICT_FP32 0x1u
#define XDK_DEPENDENT_LAUNCH 0x2u

/*
 * Multi-GPU output descriptor (no counterpart in the reference, which is single-GPU).  A column-sharded
 * projection on rank r computes columns [col0, col0 + n) of a [rows, ld] matrix; the *_peer entry points
 * store every value into all `world` destinations -- the same matrix in each rank's peer-mapped buffer
 * (xdk_peer_alloc / xdk_peer_open) -- from the kernel's epilogue, with ordinary global stores over NVLink.
 * world = 1 with ptr[0] = y, ld = n, col0 = 0 is the plain single-GPU call.
 */
#define XDK_MAX_PEERS 8
#define XDK_PEER_FLAG_BYTES 8192 /* head of every arena, reserved for the barrier flags */
typedef struct xdk_peer_out {
  void* ptr[XDK_MAX_PEERS]; /* destination matrix base on rank 0 .. world-1 (device pointers valid on THIS device) */
  int32_t world;
  int32_t reserved;
  int64_t ld;   /* elements between consecutive rows of the destination */
  int64_t col0; /* first destination column of this call's columns */
} xdk_peer_out;

/* Human-readable text for a status code (static storage). */
XDK_API const char* xdk_strerror(int status);
/* XDK_ABI_VERSION the library was built with. */
XDK_API int xdk_abi_version(void);
/* cudaError_t (as int) of the most recent failed launch on this host thread, 0 if none. */
XDK_API int xdk_last_cuda_error(void);
/*
 * Kernels that wait on mbarriers (the TMA-fed projection kernels) bound every wait by wall time; a wait
 * that gives up makes the kernel skip the work, set a bit here and return normally, so a lost copy can
 * never hang the GPU.  Returns the OR of those bits on the current device since the library was loaded
 * (bits 0-6: FP32 tile-stream projection, 8-14: W4A16 kernels, 16-22: FP32 tensor-core
 * projection; bit 31: a fault word could not be read back, treat as
 * unhealthy); 0 means no wait ever gave up.  Synchronises the device.  xdk_peer_fault_flags() is the
 * same for the multi-GPU flag barrier: bit p set = a wait on rank p ran out of time.
 */
XDK_API unsigned xdk_fault_flags(void);
XDK_API unsigned xdk_peer_fault_flags(void);
/*
 * Launches a kernel that does nothing (one warp): the cost of one kernel node on this stream or in a captured
 * graph, i.e. the floor under every per-call time the benchmarks report.  No counterpart in the reference.
 */
XDK_API int xdk_noop(unsigned flags, void* stream);
/* XDK_OK when `device` exists and is compute capability 10.x, else XDK_ERR_ARCH/ARG. */
XDK_API int xdk_device_supported(int device);

/*
 * Fused residual RMSNorm:  r = x + residual (FP32);  y = r * rsqrt(mean(r^2) + eps) * weight;
 * writes y (rounded to dtype) and residual_out = r (rounded to dtype).  The
 * UNROUNDED sum is normalised.  x, residual, y, residual_out: [rows, hidden]
 * contiguous; weight: [hidden]; all of `dtype`.  Any alignment and any
 * hidden >= 1 are accepted (16-byte aligned pointers with hidden a multiple of
 * 16 bytes take the vector path).  Outputs must not alias inputs.
 * Replaces fused_residual_rmsnorm (csrc/rmsnorm/rmsnorm_ext.cpp:10-35) ->
 * crossdsl_fused_residual_rmsnorm_cuda (csrc/rmsnorm/rmsnorm_kernel.cu:364-371).
 */
XDK_API int xdk_rmsnorm(const void* x, const void* residual, const void* weight, void* y, void* residual_out,
                int64_t rows, int64_t hidden, float eps, int dtype, void* stream);
XDK_API int xdk_rmsnorm_v2(const void* x, const void* residual, const void* weight, void* y, void* residual_out,
                   int64_t rows, int64_t hidden, float eps, int dtype, unsigned flags, void* stream);

/*
 * FP32 decode projection  y[M,N] = x[M,K] * W (+ bias[N]).
 * W is [K,N] row-major (weight_is_nk = 0) or [N,K] row-major (weight_is_nk = 1).
 * split_k in {1,2,4,8}: K is cut into split_k contiguous ranges (length
 * ceil(K/split_k) rounded up to a multiple of 32) that are reduced in a fixed
 * order inside one launch (thread-block cluster, distributed shared memory);
 * bias is added once, after the reduction.  Those kernels accumulate with FP32 FMAs.
 * split_k = 0 lets the library pick, and for 4 < M <= 16 the choice depends on `scratch`:
 *   scratch == NULL: a large projection (K % 64 == 0, K <= 16384 and, above 4096, divisible into 2, 4 or 8
 *     parts of at most 4096 that are multiples of 64; 16-byte aligned x and w, N % 4 == 0 for KN weights,
 *     K*N >= 4M) runs on the tensor cores: every operand is split into two TF32 numbers and
 *     the product formed as hi*hi + hi*lo + lo*hi with FP32 accumulation.  Against an FP64 product
 *     the relative L2 error is ~3e-6 (8e-6 on all-positive operands), below the projection's gate (1e-5), for
 *     every K the path takes (other rows stay on FP32 FMAs), but it is not the FP32-FMA result bit for bit, and
 *     an infinity in x or W yields NaN where FP32 FMAs yield an infinity (lo = v - hi is NaN for v = inf).
 *     Other shapes use the cluster kernels.
 *   scratch != NULL (device memory, >= xdk_gemv_scratch_bytes(...), 16-byte aligned, written and
 *     read inside the call only -- no initialisation, no state): strict FP32 FMA arithmetic on a
 *     persistent tile-stream kernel that deals the weight tiles evenly to all SMs.  Calls that
 *     share one scratch buffer must not overlap on the GPU.
 * Results are deterministic for a given (shape, split_k, scratch or not).  bias may be NULL.
 * M, K, N >= 1; M > 16 is processed in row tiles of 16 (the weight stream repeats per tile).
 * Replaces decode_gemv / decode_gemv_warp / decode_gemv_rows
 * (csrc/gemv/gemv_ext.cpp:57-85), decode_gemv_simt_{warp,rows} and
 * decode_gemm_tiled (csrc/gemv/gemv_simt_ext.cpp:49-83); split-K semantics as
 * src/crossdsl_kernels/triton/gemv_rows.py:47-146.
 */
XDK_API int xdk_gemv_f32(const float* x, const float* w, const float* bias, float* y,
                 int64_t m, int64_t k, int64_t n, int weight_is_nk, int split_k,
                 void* scratch, size_t scratch_bytes, void* stream);
/*
 * Version 2: the arithmetic is chosen by `flags`, not by the scratch pointer.  With XDK_STRICT_FP32 the
 * call never leaves FP32 FMA arithmetic; scratch (optional, same rules as above) then only lets a large
 * 4 < M <= 16 projection (K*N >= 48M) use the balanced tile-stream kernel instead of the cluster
 * kernels.  Without the flag, scratch is ignored whenever the tensor-core kernel takes the shape.
 */
XDK_API int xdk_gemv_f32_v2(const float* x, const float* w, const float* bias, float* y,
                    int64_t m, int64_t k, int64_t n, int weight_is_nk, int split_k,
                    void* scratch, size_t scratch_bytes, unsigned flags, void* stream);
/*
 * Introspection (no counterpart in the reference): would xdk_gemv_f32(split_k = 0, scratch = NULL) with 16-byte
 * aligned x and w run this shape on the tensor-core kernel, and with what launch?  Returns the cluster size
 * (1, 2, 4 or 8 CTAs that share each strip of columns along K) and fills out5 = {CTAs in all, K split over the
 * TMEM lane quarters (1, 2 or 4), W ring depth, dynamic shared memory in bytes, 32-column units}, or 0 when the
 * shape takes another kernel (out5 untouched), or XDK_ERR_ARG for a NULL out5.  Launches nothing.
 */
XDK_API int xdk_gemv_tc_plan(int64_t m, int64_t k, int64_t n, int weight_is_nk, int32_t* out5);
/* Bytes of scratch xdk_gemv_f32 wants for this shape on the current device (0: none needed). */
XDK_API size_t xdk_gemv_scratch_bytes(int64_t m, int64_t k, int64_t n, int weight_is_nk);

/*
 * The same projection for hosts that cannot give a kernel any workspace (no counterpart in the
 * reference).  Meant for callers that may not allocate device memory around the call -- a serving
 * loop whose memory budget went to the KV cache at start-up, a plugin interface that passes inputs
 * and outputs only.  It runs the tile-stream kernel of xdk_gemv_f32 (so 4 < M <= 16, 16-byte aligned
 * x and w, K % 4 == 0 and, for KN weights, N % 4 == 0; anything else is XDK_ERR_ARG) with its partial
 * sums in a 2.5 MB array built into the library (one copy per GPU that loads the library, held until
 * the process exits).  The array covers devices of up to 160 SMs; a device that would need more gets
 * XDK_ERR_LIMIT.  Nothing is allocated or freed: no cudaMalloc, no cudaFree, no allocating library
 * call.  The first call on a device looks the array's device address up (cudaGetSymbolAddress, with
 * that device current); make that first call before starting any stream capture.  All calls share the
 * array.  It needs no clearing -- every slot a call reads was written earlier in the same call --
 * but two calls that overlap on the GPU (different streams) race on it: serialise them.
 * Results are bit-identical to the tile-stream kernel of xdk_gemv_f32 (XDK_STRICT_FP32, split_k = 0, caller
 * scratch) -- which xdk_gemv_f32 itself selects only for K*N >= 48M; below that size it runs the cluster kernels,
 * whose summation order differs in the last bits, while this entry point runs the tile-stream kernel at every size.
 * The per-device address cache behind this call is filled without locking: concurrent first calls from several
 * host threads store the same value (harmless); after cudaDeviceReset() the cached address is stale -- do not
 * reset a device this entry point has been used on.
 */
XDK_API int xdk_gemv_f32_static_scratch(const float* x, const float* w, const float* bias, float* y,
                                        int64_t m, int64_t k, int64_t n, int weight_is_nk, void* stream);

/*
 * Fused rotary embedding + paged K/V cache append, one launch.
 * q [tokens,q_heads,head_dim], k,v [tokens,kv_heads,head_dim]; consecutive tokens of q, k, v are
 * {q,k,v}_token_stride elements apart (heads*head_dim when contiguous; larger when the three are
 * column slices of one fused QKV projection output); q_out is contiguous [tokens,q_heads,head_dim];
 * cos,sin FP32 [*, cos_width] (columns [0, rope_dim/2) are read, row = position);
 * positions, sequence_ids int64 [tokens]; page_table int64 [*, max_pages_per_seq];
 * caches [pages,page_size,kv_heads,head_dim] (cache_is_hnd = 0) or
 * [pages,kv_heads,page_size,head_dim] (cache_is_hnd = 1), same dtype as q/k/v.
 * Token t goes to physical page page_table[sequence_ids[t]][positions[t] / page_size],
 * in-page offset positions[t] % page_size.  The first rope_dim dims of each Q
 * and K head are rotated (pairs (i, i+rope_dim/2), or (2i, 2i+1) when
 * interleaved) with separately rounded FP32 multiplies and add/subtract -- no
 * fused multiply-add -- then rounded to dtype, so results are bit-identical to
 * the PyTorch reference; other dims and V are copied.  Index VALUES are not
 * checked on the device (the caller validates them at set-up); all other cache
 * slots are left untouched.
 * Replaces rope_gqa_paged_kv_append (csrc/rope_kv/rope_kv_ext.cpp:28-131) ->
 * crossdsl_rope_gqa_paged_kv_append_cuda (csrc/rope_kv/rope_kv_kernel.cu:200-275).
 */
XDK_API int xdk_rope_kv_append(const void* q, const void* k, const void* v, const float* cos, const float* sin,
                       const int64_t* positions, const int64_t* page_table, const int64_t* sequence_ids,
                       void* q_out, void* k_cache, void* v_cache,
                       int64_t tokens, int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                       int64_t cos_width, int64_t max_pages_per_seq, int64_t page_size, int64_t rope_dim,
                       int64_t q_token_stride, int64_t k_token_stride, int64_t v_token_stride,
                       int interleaved, int cache_is_hnd, int dtype, void* stream);
XDK_API int xdk_rope_kv_append_v2(const void* q, const void* k, const void* v, const float* cos, const float* sin,
                       const int64_t* positions, const int64_t* page_table, const int64_t* sequence_ids,
                       void* q_out, void* k_cache, void* v_cache,
                       int64_t tokens, int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                       int64_t cos_width, int64_t max_pages_per_seq, int64_t page_size, int64_t rope_dim,
                       int64_t q_token_stride, int64_t k_token_stride, int64_t v_token_stride,
                       int interleaved, int cache_is_hnd, int dtype, unsigned flags, void* stream);

/*
 * W4A16 projection  y[M,N] = half( x[M,K] * W^T (+ bias[N]) ), FP32 accumulation.
 * packed: uint8 [N, ceil(K/2)], two 4-bit codes per byte, even k in the low
 * nibble, value = code - 8; scales: FP16 [N, ceil(K/group_size)],
 * group_size in {32,64,128,256}; W[n][k] = half(float(value) * float(scale)),
 * that rounding included.  x, bias (nullable), y are FP16.  1 <= M <= 16.
 * Replaces linear_out (csrc/w4a16/w4a16_ext.cpp:7-39) -> w4a16_launch
 * (csrc/w4a16/w4a16_kernel.cu:45-63).
 */
XDK_API int xdk_w4a16(const void* x, const uint8_t* packed, const void* scales, const void* bias, void* y,
              int64_t m, int64_t k, int64_t n, int group_size, void* stream);
XDK_API int xdk_w4a16_v2(const void* x, const uint8_t* packed, const void* scales, const void* bias, void* y,
                 int64_t m, int64_t k, int64_t n, int group_size, unsigned flags, void* stream);

/*
 * The two ops that follow the path in a decoder layer (no counterpart in the reference, whose chain stops at
 * the append and at the up+gate projection; expectations are this library's own FP32 restatements).
 *
 * xdk_paged_decode_attention: one query token per sequence against the paged K/V cache the append wrote.
 *   out[t][h] = sum_j softmax_j(scale * q[t][h] . K[j][h / G]) * V[j][h / G],  j = 0 .. positions[t] (the token's own
 *   K/V are in the cache already), G = q_heads / kv_heads in {1, 2, 4, 8}, head_dim in {64, 128, 256}; q and out
 *   [tokens, q_heads, head_dim] contiguous; caches, positions, page_table, sequence_ids and the address
 *   translation exactly as in xdk_rope_kv_append.  FP32 scores, softmax and accumulation.  context_hint: the longest
 *   context the caller expects (bounds how finely the context is split across CTAs; <= 0: long).  One launch, no
 *   scratch: the slices of a (token, KV head) are merged through distributed shared memory in a fixed order.
 * xdk_swiglu: out[r][j] = silu(upgate[r][width + j]) * upgate[r][j] for j < width -- columns [0, width) of the fused
 *   projection are "up", [width, 2 width) "gate"; in_ld / out_ld: elements between rows.
 */
XDK_API int xdk_paged_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int64_t* positions,
                               const int64_t* page_table, const int64_t* sequence_ids, void* out, int64_t tokens,
                               int64_t q_heads, int64_t kv_heads, int64_t head_dim, int64_t max_pages_per_seq,
                               int64_t page_size, int cache_is_hnd, float scale, int64_t context_hint, int dtype,
                               unsigned flags, void* stream);
XDK_API int xdk_swiglu(const void* upgate, void* out, int64_t rows, int64_t width, int64_t in_ld, int64_t out_ld, int dtype,
               unsigned flags, void* stream);
/*
 * The same two ops with the result stored into the same place of every rank's peer-mapped matrix (see
 * xdk_gemv_f32_peer): out_dst->ld is the row pitch of the full-width matrix in elements, out_dst->col0 the first
 * column of this rank's share ([tokens, q_heads * head_dim] for the attention output, [rows, width] for SwiGLU).
 * A decode layer sharded by KV head (attention) and by MLP column (up and gate shards side by side on a rank)
 * needs no other exchange than these two stores and a flag barrier after each.
 */
XDK_API int xdk_paged_decode_attention_peer(const void* q, const void* k_cache, const void* v_cache, const int64_t* positions,
                                    const int64_t* page_table, const int64_t* sequence_ids, const xdk_peer_out* out_dst,
                                    int64_t tokens, int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                                    int64_t max_pages_per_seq, int64_t page_size, int cache_is_hnd, float scale,
                                    int64_t context_hint, int dtype, unsigned flags, void* stream);
XDK_API int xdk_swiglu_peer(const void* upgate, const xdk_peer_out* out_dst, int64_t rows, int64_t width, int64_t in_ld,
                    int dtype, unsigned flags, void* stream);


/*
 * Symmetric INT4 quantisation on the device, into the format xdk_w4a16 reads: weight [n, k] row-major of
 * `dtype` (FP32, BF16 or FP16) -> packed uint8 [n, ceil(k/2)] and FP16 scales [n, ceil(k/group_size)].
 * Per (row, group): scale = half(max|w| / 7) (at least 2^-24; 1 for an all-zero group), rounded to FP16
 * BEFORE q = clamp(round-half-even(w / scale), -7, 7) is chosen; code = q + 8.  Packed bytes and scales are
 * bit-identical to the host function.  *status (device int32, zero it first) receives the OR of
 * 1 = a weight is not finite, 2 = a scale is not representable in FP16, 4 = a dequantised weight is not
 * representable in FP16 -- the three conditions the host function raises on; read it after the stream drained.
 * Replaces the set-up step quantize_int4 (src/crossdsl_kernels/quantization.py:39-63) for weights that
 * already live on the device.
 */
XDK_API int xdk_quantize_int4(const void* weight, int dtype, int64_t n, int64_t k, int group_size, uint8_t* packed,
                      void* scales, int* status, void* stream);

/*
 * Multi-GPU plumbing, one process per GPU on one node (no upstream counterpart).
 * xdk_peer_alloc: a zeroed cudaMalloc arena of `bytes` (>= XDK_PEER_FLAG_BYTES; the head of that size holds the
 *   barrier flags, payload starts behind it).  This and xdk_peer_free are the only entry points that allocate.
 * xdk_peer_export / xdk_peer_open / xdk_peer_close: the arena as a 64-byte CUDA IPC handle, and another
 *   process's handle mapped into this one (peer access is enabled on first use).
 * xdk_peer_barrier: launched by EVERY rank on its stream after the kernels that stored into the peers' arenas:
 *   publishes this rank's next epoch for `site` (0..63; use one site per exchange point of a step) to every
 *   arena and waits until all `world` ranks have published it, at most timeout_us microseconds (0: one second).
 *   arenas[p] = rank p's arena as mapped here (arenas[rank] = the local one).  A wait that runs out sets bit p
 *   of xdk_peer_fault_flags() and the kernel returns normally.  Epochs live on the device, so the launch can be
 *   captured in a CUDA graph and replayed -- by all ranks equally often.
 */
XDK_API int xdk_peer_alloc(size_t bytes, void** ptr);
XDK_API int xdk_peer_free(void* ptr);
XDK_API int xdk_peer_export(void* ptr, void* handle64);
XDK_API int xdk_peer_open(const void* handle64, void** ptr);
XDK_API int xdk_peer_close(void* ptr);
XDK_API int xdk_peer_barrier(void* const* arenas, int rank, int world, int site, unsigned timeout_us, unsigned flags,
                     void* stream);
/* The projections and the append with their output (rotated Q for the append) stored into every rank's buffer. */
XDK_API int xdk_gemv_f32_peer(const float* x, const float* w, const float* bias, const xdk_peer_out* y,
                      int64_t m, int64_t k, int64_t n, int weight_is_nk, int split_k,
                      void* scratch, size_t scratch_bytes, unsigned flags, void* stream);
XDK_API int xdk_w4a16_peer(const void* x, const uint8_t* packed, const void* scales, const void* bias,
                   const xdk_peer_out* y, int64_t m, int64_t k, int64_t n, int group_size, unsigned flags, void* stream);
XDK_API int xdk_rope_kv_append_peer(const void* q, const void* k, const void* v, const float* cos, const float* sin,
                       const int64_t* positions, const int64_t* page_table, const int64_t* sequence_ids,
                       const xdk_peer_out* q_out, void* k_cache, void* v_cache,
                       int64_t tokens, int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                       int64_t cos_width, int64_t max_pages_per_seq, int64_t page_size, int64_t rope_dim,
                       int64_t q_token_stride, int64_t k_token_stride, int64_t v_token_stride,
                       int interleaved, int cache_is_hnd, int dtype, unsigned flags, void* stream);

/*
 * Multi-GPU helper with no upstream counterpart (upstream is single-GPU): after an all-gather of
 * column shards, `gathered` holds [world, rows, cols_per_rank] (rank-major); this writes the
 * row-major matrix out[rows, world * cols_per_rank] in which rank r owns columns
 * [r * cols_per_rank, (r + 1) * cols_per_rank).  elem_bytes in {1,2,4,8}.  out must not alias gathered.
 */
XDK_API int xdk_unshard_columns(const void* gathered, void* out, int64_t world, int64_t rows,
                                int64_t cols_per_rank, int elem_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* XDK_B200_H_ */
