// Row movement for any dtype and trailing shape: a row is `row_bytes` contiguous bytes.
//
//   gather   out[i, :] = map[i] >= 0 ? x[map[i], :] : 0      (slot padding, restore, shard select)
//   scatter  out[rows[i], :] = x[i, :]                        (adjoint of a unique-row gather)
//
// Replaces the reference's per-element Triton copies (vsa_kernels.py:11-26, 66-83, 119-132) with
// 16-byte vector copies: consecutive threads move consecutive vectors of one row, so both sides
// are coalesced.  Rows of 32 vectors or more get a warp each; narrower rows (position ids, small
// trailing shapes) use one thread per vector.  Offsets are 64-bit; tensors beyond 2^31 elements
// are fine.
#include "vsa_common.cuh"
#include "vsa_kernels.h"

namespace vsa {

namespace {

template <typename V>
__global__ void row_gather_kernel(const V* __restrict__ x, const int64_t* __restrict__ map, V* __restrict__ out,
                                  long long total, long long vecs_per_row) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long row = i / vecs_per_row, v = i - row * vecs_per_row;
  const long long src = map[row];
  V value{};
  if (src >= 0) value = x[src * vecs_per_row + v];
  out[i] = value;
}

template <typename V>
__global__ void row_scatter_kernel(const V* __restrict__ x, const int64_t* __restrict__ rows, V* __restrict__ out,
                                   long long total, long long vecs_per_row) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long row = i / vecs_per_row, v = i - row * vecs_per_row;
  const long long dst = rows[row];
  if (dst >= 0) out[dst * vecs_per_row + v] = x[i];
}

struct alignas(16) Vec16 { uint32_t w[4]; };

// Wide rows (at least 32 vectors): one warp per row.  The map entry is read once per row, there
// is no index division, and every lane keeps up to four independent 16-byte loads in flight.
template <typename V, bool kScatter>
__global__ void __launch_bounds__(256) wide_row_kernel(const V* __restrict__ x, const int64_t* __restrict__ map,
                                                       V* __restrict__ out, long long rows, int vecs_per_row) {
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long other = map[row];
  const V* src = x + (kScatter ? row : other) * vecs_per_row;
  V* dst = out + (kScatter ? other : row) * vecs_per_row;
  if (other < 0) {
    if (!kScatter)
      for (int v = lane; v < vecs_per_row; v += 32) dst[v] = V{};
    return;
  }
  int v = lane;
  for (; v + 96 < vecs_per_row; v += 128) {
    const V a = src[v], b = src[v + 32], c = src[v + 64], d = src[v + 96];
    dst[v] = a, dst[v + 32] = b, dst[v + 64] = c, dst[v + 96] = d;
  }
  for (; v < vecs_per_row; v += 32) dst[v] = src[v];
}

// Widest power-of-two vector (<= 16 bytes) that divides the row and both base addresses.
int vector_bytes(const void* a, const void* b, long long row_bytes) {
  const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                         static_cast<uintptr_t>(row_bytes);
  int width = 16;
  while (width > 1 && (bits & (width - 1))) width >>= 1;
  return width;
}

template <typename V, bool kScatter>
cudaError_t launch(const void* x, const int64_t* map, void* out, long long rows, long long row_bytes,
                   cudaStream_t stream) {
  const long long vecs = row_bytes / static_cast<long long>(sizeof(V));
  const long long total = rows * vecs;
  if (total == 0) return cudaSuccess;
  if (vecs >= 32 && vecs <= 0x7fffffffLL) {
    const long long ctas = (rows + 7) / 8;  // eight warps, one row each
    if (ctas > 0x7fffffffLL) return cudaErrorInvalidValue;
    wide_row_kernel<V, kScatter><<<static_cast<unsigned>(ctas), 256, 0, stream>>>(
        static_cast<const V*>(x), map, static_cast<V*>(out), rows, static_cast<int>(vecs));
    return cudaGetLastError();
  }
  const int threads = 256;
  const long long blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
  if (kScatter)
    row_scatter_kernel<V><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        static_cast<const V*>(x), map, static_cast<V*>(out), total, vecs);
  else
    row_gather_kernel<V><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        static_cast<const V*>(x), map, static_cast<V*>(out), total, vecs);
  return cudaGetLastError();
}

template <bool kScatter>
cudaError_t dispatch(const void* x, const int64_t* map, void* out, long long rows, long long row_bytes,
                     cudaStream_t stream) {
  switch (vector_bytes(x, out, row_bytes)) {
    case 16: return launch<Vec16, kScatter>(x, map, out, rows, row_bytes, stream);
    case 8: return launch<uint64_t, kScatter>(x, map, out, rows, row_bytes, stream);
    case 4: return launch<uint32_t, kScatter>(x, map, out, rows, row_bytes, stream);
    case 2: return launch<uint16_t, kScatter>(x, map, out, rows, row_bytes, stream);
    default: return launch<uint8_t, kScatter>(x, map, out, rows, row_bytes, stream);
  }
}

}  // namespace

cudaError_t launch_row_gather(const void* x, const int64_t* map, void* out, long long out_rows,
                              long long row_bytes, cudaStream_t stream) {
  return dispatch<false>(x, map, out, out_rows, row_bytes, stream);
}

cudaError_t launch_row_scatter(const void* x, const int64_t* rows, void* out, long long in_rows,
                               long long row_bytes, cudaStream_t stream) {
  return dispatch<true>(x, rows, out, in_rows, row_bytes, stream);
}

}  // namespace vsa
