// Ring (context-parallel) helpers.
//
//   partition_indices  splits every routing row of global block ids into one list per owner rank,
//                      holding owner-local block ids in the original (ascending) order, tails
//                      zeroed (reference vsa_kernels.py:285-353).
//   merge_partial      online-softmax merge of one ring step's normalised partial output and LSE
//                      into the running FP32 output and LSE; empty rows (-inf) contribute nothing
//                      (reference vsa_kernels.py:375-397).  One warp owns a (slot, head) row, so the
//                      LSE is updated in place without a second buffer.
#include "vsa_common.cuh"
#include "vsa_kernels.h"

namespace vsa {

namespace {

constexpr int kPartThreads = 128;

__global__ void __launch_bounds__(kPartThreads) partition_kernel(
    const int32_t* __restrict__ index, const int32_t* __restrict__ counts,
    const int64_t* __restrict__ global_to_gather, int32_t* __restrict__ out_lists,
    int32_t* __restrict__ out_counts, int capacity, int out_capacity, int peer_blocks, long long list_stride,
    long long count_stride) {
  __shared__ int partial[kPartThreads];
  __shared__ int s_total;
  const long long row = blockIdx.x;
  const int peer = blockIdx.y;
  const int n = counts[row];
  const int32_t* src = index + row * capacity;
  const int per = (n + kPartThreads - 1) / kPartThreads;
  const int begin = min(n, static_cast<int>(threadIdx.x) * per), end = min(n, begin + per);
  int mine = 0;
  for (int i = begin; i < end; ++i) mine += (global_to_gather[src[i]] / peer_blocks) == peer;
  partial[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    int running = 0;
    for (int t = 0; t < kPartThreads; ++t) {
      const int x = partial[t];
      partial[t] = running;
      running += x;
    }
    out_counts[peer * count_stride + row] = running;
    s_total = running;
  }
  __syncthreads();
  int32_t* dst = out_lists + peer * list_stride + row * out_capacity;
  int cursor = partial[threadIdx.x];
  for (int i = begin; i < end; ++i) {
    const long long mapped = global_to_gather[src[i]];
    if (mapped / peer_blocks == peer) {
      if (cursor < out_capacity) dst[cursor] = static_cast<int32_t>(mapped % peer_blocks);
      ++cursor;
    }
  }
  for (int i = s_total + threadIdx.x; i < out_capacity; i += kPartThreads) dst[i] = 0;
}

// bounds[row][c] = first position of the row's ascending list whose block id is >= c * chunk_blocks
// (c = 0 .. chunks - 1); bounds[row][chunks] = the row's count.  One thread per (row, c).
__global__ void list_bounds_kernel(const int32_t* __restrict__ lists, const int32_t* __restrict__ counts,
                                   long long rows, int capacity, int chunk_blocks, int chunks,
                                   int32_t* __restrict__ bounds) {
  const long long id = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long row = id / (chunks + 1);
  const int c = static_cast<int>(id - row * (chunks + 1));
  if (row >= rows) return;
  const int n = min(counts[row], capacity);
  int lo = 0, hi = n;
  if (c < chunks) {
    const long long first = static_cast<long long>(c) * chunk_blocks;
    const int32_t* list = lists + row * capacity;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (list[mid] < first) lo = mid + 1; else hi = mid;
    }
  } else {
    lo = n;
  }
  bounds[row * (chunks + 1) + c] = lo;
}

__global__ void merge_partial_kernel(float* __restrict__ out, float* __restrict__ lse,
                                     const __nv_bfloat16* __restrict__ part, const float* __restrict__ part_lse,
                                     long long slots, int heads) {
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= slots * heads) return;
  const long long slot = warp / heads;
  const int head = static_cast<int>(warp - slot * heads);
  const long long l_off = static_cast<long long>(head) * slots + slot;
  const float old_l = lse[l_off], new_l = part_lse[l_off];
  float top = fmaxf(old_l, new_l);
  if (top == -INFINITY) top = 0.f;
  const float w_old = expf(old_l - top), w_new = expf(new_l - top);
  const float denom = w_old + w_new;
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  const long long off = (slot * heads + head) * kDim + lane * 4;
  const float4 o = *reinterpret_cast<const float4*>(out + off);
  const uint2 raw = *reinterpret_cast<const uint2*>(part + off);
  const float2 p01 = unpack_bf16(raw.x), p23 = unpack_bf16(raw.y);
  float4 r;
  r.x = ((w_old > 0.f ? o.x * w_old : 0.f) + (w_new > 0.f ? p01.x * w_new : 0.f)) * inv;
  r.y = ((w_old > 0.f ? o.y * w_old : 0.f) + (w_new > 0.f ? p01.y * w_new : 0.f)) * inv;
  r.z = ((w_old > 0.f ? o.z * w_old : 0.f) + (w_new > 0.f ? p23.x * w_new : 0.f)) * inv;
  r.w = ((w_old > 0.f ? o.w * w_old : 0.f) + (w_new > 0.f ? p23.y * w_new : 0.f)) * inv;
  *reinterpret_cast<float4*>(out + off) = r;
  __syncwarp();
  if (lane == 0) lse[l_off] = top + logf(denom);
}

}  // namespace

cudaError_t launch_partition_indices(const int32_t* index, const int32_t* counts, const int64_t* global_to_gather,
                                     int32_t* out_lists, int32_t* out_counts, long long rows, int capacity,
                                     int out_capacity, int ring_size, int peer_blocks, long long list_stride,
                                     long long count_stride, cudaStream_t stream) {
  if (rows == 0 || ring_size == 0) return cudaSuccess;
  dim3 grid(static_cast<unsigned>(rows), ring_size);
  partition_kernel<<<grid, kPartThreads, 0, stream>>>(index, counts, global_to_gather, out_lists, out_counts, capacity,
                                                      out_capacity, peer_blocks, list_stride, count_stride);
  return cudaGetLastError();
}

cudaError_t launch_list_bounds(const int32_t* lists, const int32_t* counts, long long rows, int capacity,
                               int chunk_blocks, int chunks, int32_t* bounds, cudaStream_t stream) {
  const long long threads = rows * (chunks + 1);
  if (threads == 0) return cudaSuccess;
  list_bounds_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(lists, counts, rows, capacity,
                                                                                      chunk_blocks, chunks, bounds);
  return cudaGetLastError();
}

cudaError_t launch_merge_partial(float* out, float* lse, const __nv_bfloat16* part, const float* part_lse,
                                 long long slots, int heads, cudaStream_t stream) {
  const long long warps = slots * heads;
  if (warps == 0) return cudaSuccess;
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  merge_partial_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(out, lse, part, part_lse, slots, heads);
  return cudaGetLastError();
}

}  // namespace vsa
