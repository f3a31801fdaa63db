// Column un-sharding after an all-gather.  A rank-major gather of per-rank shards [rows, cols] lands
// as [world, rows, cols]; consumers want the row-major matrix [rows, world * cols] in which rank r
// owns columns [r * cols, (r + 1) * cols).  One 16-byte vector per thread when the shapes allow.
#include "common.cuh"

namespace xdk {
namespace {

template <typename V>
__global__ void __launch_bounds__(256)
unshard_kernel(const V* __restrict__ gathered, V* __restrict__ out, int world, int rows, int vec_per_row) {
  const int64_t total = static_cast<int64_t>(world) * rows * vec_per_row;
  for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
    const int v = static_cast<int>(i % vec_per_row);
    const int64_t rr = i / vec_per_row;
    const int row = static_cast<int>(rr % rows), rank = static_cast<int>(rr / rows);
    out[(static_cast<int64_t>(row) * world + rank) * vec_per_row + v] = gathered[i];
  }
}

}  // namespace
}  // namespace xdk

extern "C" int xdk_unshard_columns(const void* gathered, void* out, int64_t world, int64_t rows, int64_t cols_per_rank,
                                   int elem_bytes, void* stream) {
  using namespace xdk;
  if (!gathered || !out || world < 1 || rows < 1 || cols_per_rank < 1) return XDK_ERR_ARG;
  if (!(elem_bytes == 1 || elem_bytes == 2 || elem_bytes == 4 || elem_bytes == 8)) return XDK_ERR_ARG;
  if (world > 65535 || rows > 2147483647LL || cols_per_rank * elem_bytes > 2147483647LL) return XDK_ERR_LIMIT;
  if (int st = require_sm100()) return st;
  const int64_t row_bytes = cols_per_rank * elem_bytes;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool vec = row_bytes % 16 == 0 && aligned16(gathered) && aligned16(out);
  const int64_t per_row = vec ? row_bytes / 16 : row_bytes;
  const int64_t total = world * rows * per_row;
  const unsigned grid = static_cast<unsigned>(total / 256 + 1 > 148 * 8 ? 148 * 8 : total / 256 + 1);
  if (vec)
    return launch(unshard_kernel<U4>, dim3(grid), dim3(256), 0, s, 1u, static_cast<const U4*>(gathered),
                  static_cast<U4*>(out), static_cast<int>(world), static_cast<int>(rows), static_cast<int>(per_row));
  return launch(unshard_kernel<unsigned char>, dim3(grid), dim3(256), 0, s, 1u,
                static_cast<const unsigned char*>(gathered), static_cast<unsigned char*>(out), static_cast<int>(world),
                static_cast<int>(rows), static_cast<int>(per_row));
}
