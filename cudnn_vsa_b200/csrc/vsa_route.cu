// Routing: per (head, query block) choose the `keep` KV blocks of one video region with the
// highest pooled scores and list them in ascending block order.
//
//   route_scores_kernel   scores[h, q, j] = q_mean[q, h, :] . k_mean[j, h, :] in true FP32 on
//                         the CUDA cores (no TF32, unscaled), 128 x 128 tiles, 8 x 8 per thread.
//   route_select_kernel   one CTA per row: exact radix select of the keep-th largest score
//                         (four 8-bit passes over order-preserving keys, the digit found with a
//                         block-wide prefix sum), then an ordered compaction, so ids come out
//                         ascending and ties at the threshold go to the lowest block ids.
//
// Replaces the reference's per-region SGEMM + topk + sort (vsa_core.py:61-72).
#include "vsa_common.cuh"
#include "vsa_kernels.h"

namespace vsa {

namespace {

constexpr int kTile = 128;   // query rows and KV columns of a score tile
constexpr int kSlice = 32;   // head dims staged per shared-memory round

// 128 x 128 score tiles, 8 x 8 per thread: per head dim a thread reads two float4 of each operand
// (shared-memory broadcasts within a warp) for 64 FMAs, which balances the shared-memory and FMA
// pipes; the 64 x 64 / 4 x 4 form spent two thirds of its time on operand loads.  A thread's rows
// and columns are split in two groups of four, 64 apart, so that a warp's loads stay contiguous.
__global__ void __launch_bounds__(256) route_scores_kernel(const float* __restrict__ q_mean,
                                                           const float* __restrict__ k_mean, int heads,
                                                           int head0, RouteSpan span, float* __restrict__ scores) {
  // Operand tiles stored [d][row] so that a thread's 4 rows are one 16-byte shared load.
  __shared__ __align__(16) float qs[kSlice][kTile];
  __shared__ __align__(16) float ks[kSlice][kTile];
  const int nq = span.q_end - span.q_begin, nk = span.kv_last - span.kv_first;
  const int q0 = blockIdx.y * kTile, k0 = blockIdx.x * kTile;
  const int head = head0 + blockIdx.z;
  const long long width = static_cast<long long>(heads) * kDim;
  const int tq = (threadIdx.x / 16) * 4, tk = (threadIdx.x % 16) * 4;  // + 64 for the second group
  float acc[8][8] = {};
  for (int d0 = 0; d0 < kDim; d0 += kSlice) {
    __syncthreads();
    // Consecutive threads take consecutive rows: the transposed shared stores are conflict-free.
    for (int i = threadIdx.x; i < kTile * (kSlice / 4); i += blockDim.x) {
      const int r = i % kTile, d4 = i / kTile;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
      if (q0 + r < nq)
        a = __ldg(reinterpret_cast<const float4*>(
            q_mean + (static_cast<long long>(span.q_begin + q0 + r) + span.q_mean_offset) * width + head * kDim + d0) + d4);
      if (k0 + r < nk)
        b = __ldg(reinterpret_cast<const float4*>(
            k_mean + (static_cast<long long>(span.kv_first + k0 + r) + span.k_mean_offset) * width + head * kDim + d0) + d4);
      qs[4 * d4][r] = a.x, qs[4 * d4 + 1][r] = a.y, qs[4 * d4 + 2][r] = a.z, qs[4 * d4 + 3][r] = a.w;
      ks[4 * d4][r] = b.x, ks[4 * d4 + 1][r] = b.y, ks[4 * d4 + 2][r] = b.z, ks[4 * d4 + 3][r] = b.w;
    }
    __syncthreads();
#pragma unroll 4
    for (int d = 0; d < kSlice; ++d) {
      const float4 a0 = *reinterpret_cast<const float4*>(&qs[d][tq]);
      const float4 a1 = *reinterpret_cast<const float4*>(&qs[d][tq + 64]);
      const float4 b0 = *reinterpret_cast<const float4*>(&ks[d][tk]);
      const float4 b1 = *reinterpret_cast<const float4*>(&ks[d][tk + 64]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
  }
  float* out = scores + static_cast<long long>(blockIdx.z) * nq * nk;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int qi = q0 + tq + (i & 3) + (i >> 2) * 64;
    if (qi >= nq) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int kj = k0 + tk + (j & 3) + (j >> 2) * 64;
      if (kj < nk) out[static_cast<long long>(qi) * nk + kj] = acc[i][j];
    }
  }
}

VSA_DEVICE uint32_t order_key(float f) {
  const uint32_t bits = __float_as_uint(f);
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

// Inclusive prefix sum of `v` over the 256 threads of the CTA, in thread order (warp shuffles plus
// one exchange of the eight warp totals through `totals`).  Every thread must call it.
VSA_DEVICE int block_prefix_sum(int v, int* totals) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, v, off);
    if (lane >= off) v += up;
  }
  __syncthreads();  // the previous use of `totals` has been read
  if (lane == 31) totals[warp] = v;
  __syncthreads();
  for (int w = 0; w < warp; ++w) v += totals[w];
  return v;
}

__global__ void __launch_bounds__(256) route_select_kernel(const float* __restrict__ scores, int head0,
                                                           RouteSpan span, int32_t* __restrict__ indices,
                                                           long long index_head_stride, int capacity) {
  extern __shared__ uint32_t keys[];
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  __shared__ int totals[8];
  const int nq = span.q_end - span.q_begin, n = span.kv_last - span.kv_first;
  const int qi = blockIdx.x, head = head0 + blockIdx.y;
  const float* row = scores + (static_cast<long long>(blockIdx.y) * nq + qi) * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) keys[i] = order_key(row[i]);
  if (threadIdx.x == 0) s_prefix = 0, s_remaining = span.keep;
  __syncthreads();
  uint32_t known = 0;
  for (int pass = 3; pass >= 0; --pass) {
    hist[threadIdx.x] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const int remaining = s_remaining;
    for (int i = threadIdx.x; i < n; i += blockDim.x)
      if ((keys[i] & known) == prefix) atomicAdd(&hist[(keys[i] >> (8 * pass)) & 255], 1);
    __syncthreads();
    // Thread t owns digit 255 - t, so the running sum counts the candidates whose digit is at
    // least its own.  The digit of the keep-th largest key is the one where that count first
    // reaches `remaining`; exactly one thread (with a non-empty bin) sees the crossing.
    const int mine = hist[255 - threadIdx.x];
    const int at_least = block_prefix_sum(mine, totals), above = at_least - mine;
    if (above < remaining && remaining <= at_least) {
      s_remaining = remaining - above;
      s_prefix = prefix | (static_cast<uint32_t>(255 - threadIdx.x) << (8 * pass));
    }
    known |= 0xFFu << (8 * pass);
    __syncthreads();
  }
  const uint32_t threshold = s_prefix;  // key of the keep-th largest score
  const int ties = s_remaining;         // how many scores equal to it are taken, lowest ids first
  const int per = (n + blockDim.x - 1) / blockDim.x;
  const int begin = min(n, static_cast<int>(threadIdx.x) * per), end = min(n, begin + per);
  int gt = 0, eq = 0;
  for (int i = begin; i < end; ++i) gt += keys[i] > threshold, eq += keys[i] == threshold;
  // Ordered compaction: entries before this thread's segment that are above / at the threshold.
  int before_gt = block_prefix_sum(gt, totals) - gt;
  int before_eq = block_prefix_sum(eq, totals) - eq;
  int32_t* out = indices + static_cast<long long>(head) * index_head_stride +
                 static_cast<long long>(span.q_begin + qi) * capacity + span.cursor;
  for (int i = begin; i < end; ++i) {
    const uint32_t key = keys[i];
    if (key > threshold) {
      out[before_gt + min(before_eq, ties)] = span.kv_first + i;
      ++before_gt;
    } else if (key == threshold) {
      if (before_eq < ties) out[before_gt + before_eq] = span.kv_first + i;
      ++before_eq;
    }
  }
}

}  // namespace

// `scores` is caller-provided scratch of at least head_chunk * rows * region floats; heads are
// processed head_chunk at a time so the scratch stays bounded.
cudaError_t launch_route_chunk(const float* q_mean, const float* k_mean, int heads, int head0, int head_chunk,
                               const RouteSpan& span, float* scores, int32_t* indices,
                               long long index_head_stride, int capacity, cudaStream_t stream) {
  const int nq = span.q_end - span.q_begin, n = span.kv_last - span.kv_first;
  if (nq <= 0 || n <= 0 || head_chunk <= 0) return cudaSuccess;
  dim3 grid((n + kTile - 1) / kTile, (nq + kTile - 1) / kTile, head_chunk);
  route_scores_kernel<<<grid, 256, 0, stream>>>(q_mean, k_mean, heads, head0, span, scores);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  const size_t smem = static_cast<size_t>(n) * sizeof(uint32_t);
  if (smem > 48 * 1024) {
    err = cudaFuncSetAttribute(route_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) return err;
  }
  route_select_kernel<<<dim3(nq, head_chunk), 256, smem, stream>>>(scores, head0, span, indices, index_head_stride,
                                                                   capacity);
  return cudaGetLastError();
}

}  // namespace vsa
