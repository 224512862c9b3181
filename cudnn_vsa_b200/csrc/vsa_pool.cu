// HBM-bound block kernels.  A CTA owns up to 128 16-byte column chunks of one 64-slot block and
// splits the block's slots over two or more groups of threads, so that every thread keeps
// several independent 16-byte loads in flight and a block of few heads still fills its SM;
// wide rows (many heads) are split over several CTAs per block.
//
//   slots_pool   reads Q, K, V rows once through the slot map, writes the zero-padded slot
//                tensors and the FP32 block means (sum of the slots / max(size, 1)) plus their
//                BF16 rounding placed at the block's row of the coarse streams.  Fuses the
//                reference's three slot gathers with its pooling reduction
//                (vsa_kernels.py:66-83, 119-158, 161-188; vsa.py:96-104).
//   merge_bwd    adjoint of `out = fine + gate * coarse[block]` fused with the gather of dO into
//                slots and with delta = rowsum(dO * O_fine) that the fine backward needs
//                (vsa_kernels.py:204-246; vsa_core.py:23-30 consumes O and dO).
#include "vsa_common.cuh"
#include "vsa_kernels.h"

namespace vsa {

namespace {

constexpr int kChunk = 8;          // BF16 elements per 16-byte chunk
constexpr int kCtaChunks = 128;    // column chunks per CTA at most (a multiple of 16 = one head)
constexpr int kCtaThreads = 256;   // threads per CTA at most

VSA_DEVICE void accumulate(float (&acc)[8], const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = unpack_bf16(w[e]);
    acc[2 * e] += f.x;
    acc[2 * e + 1] += f.y;
  }
}

// Launch shape shared by the block kernels: grid (blocks, column parts), `cols` chunks per CTA
// and `groups` slot groups (threads = cols * groups; thread = (group, column chunk)).
struct BlockShape {
  int cols, groups, parts;
};
BlockShape block_shape(int chunks) {
  BlockShape s;
  s.parts = (chunks + kCtaChunks - 1) / kCtaChunks;
  s.cols = (chunks + s.parts - 1) / s.parts;
  s.cols = ((s.cols + 15) / 16) * 16;        // whole heads, so the 16-lane head sums stay together
  s.groups = 1;  // a power of two (it divides the 64 slots), at most 8
  while (s.groups < 8 && s.cols * s.groups * 2 <= kCtaThreads) s.groups *= 2;
  return s;
}

__global__ void __launch_bounds__(kCtaThreads) slots_pool_kernel(const PoolParams p, int cols, int groups) {
  __shared__ long long rows[kBlock];
  extern __shared__ float partial[];  // [groups - 1][cols][24] sums of the other slot groups
  const long long block = blockIdx.x;
  for (int i = threadIdx.x; i < kBlock; i += blockDim.x) {
    const long long slot = block * kBlock + i;
    rows[i] = p.slot_row != nullptr ? p.slot_row[slot] : slot;
  }
  __syncthreads();
  const int chunks = p.width / kChunk;
  const int local = threadIdx.x % cols, group = threadIdx.x / cols;
  const int c = blockIdx.y * cols + local;
  const bool active = c < chunks;
  const int size = p.sizes[block];
  const int per = kBlock / groups;  // slots of this thread: [group * per, group * per + per)
  const uint4* src[3] = {reinterpret_cast<const uint4*>(p.q), reinterpret_cast<const uint4*>(p.k),
                         reinterpret_cast<const uint4*>(p.v)};
  uint4* dst[3] = {reinterpret_cast<uint4*>(p.q_slots), reinterpret_cast<uint4*>(p.k_slots),
                   reinterpret_cast<uint4*>(p.v_slots)};
  float acc[3][8] = {};
  // Input rows may be strided (q, k, v interleaved in one projection output): 16-byte units.
  const long long in_row = p.in_row_stride / kChunk;
  const long long in_col = (c / (kDim / kChunk)) * (p.in_head_stride / kChunk) + c % (kDim / kChunk);
  if (active) {
#pragma unroll 8
    for (int s = group * per; s < (group + 1) * per; ++s) {
      const long long row = rows[s];
      const long long out = (block * kBlock + s) * chunks + c;
#pragma unroll
      for (int t = 0; t < 3; ++t) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row >= 0) v = __ldg(src[t] + row * in_row + in_col);
        if (dst[t] != nullptr) dst[t][out] = v;
        accumulate(acc[t], v);
      }
    }
  }
  if (p.mean_f32 == nullptr && p.mean_bf16 == nullptr) return;
  if (groups > 1) {
    if (group > 0) {
      float* mine = partial + (static_cast<size_t>(group - 1) * cols + local) * 24;
#pragma unroll
      for (int t = 0; t < 3; ++t)
#pragma unroll
        for (int e = 0; e < 8; ++e) mine[t * 8 + e] = acc[t][e];
    }
    __syncthreads();
    if (group > 0) return;
    for (int g = 1; g < groups; ++g) {
      const float* other = partial + (static_cast<size_t>(g - 1) * cols + local) * 24;
#pragma unroll
      for (int t = 0; t < 3; ++t)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[t][e] += other[t * 8 + e];
    }
  }
  if (!active) return;
  const float inv = 1.f / static_cast<float>(size > 1 ? size : 1);
  const long long coarse_row = (p.block_coarse != nullptr && p.mean_bf16 != nullptr) ? p.block_coarse[block] : -1;
#pragma unroll
  for (int t = 0; t < 3; ++t) {
    float mean[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) mean[e] = acc[t][e] * inv;
    if (p.mean_f32 != nullptr) {
      float4* m = reinterpret_cast<float4*>(p.mean_f32 + (t * p.blocks + block) * p.width + c * kChunk);
      m[0] = make_float4(mean[0], mean[1], mean[2], mean[3]);
      m[1] = make_float4(mean[4], mean[5], mean[6], mean[7]);
    }
    if (coarse_row >= 0) {
      uint4* m = reinterpret_cast<uint4*>(p.mean_bf16 + (t * p.coarse_rows + coarse_row) * p.width + c * kChunk);
      *m = make_uint4(pack_bf16(mean[0], mean[1]), pack_bf16(mean[2], mean[3]), pack_bf16(mean[4], mean[5]),
                      pack_bf16(mean[6], mean[7]));
    }
  }
}

// Sum over the 16 consecutive lanes that hold one head's 128 columns.
VSA_DEVICE float head_sum(float x) {
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
  return x;
}

__global__ void __launch_bounds__(kCtaThreads) merge_bwd_kernel(const MergeBwdParams p, int cols, int groups) {
  __shared__ long long rows[kBlock];
  extern __shared__ float partial[];  // [groups - 1][cols][8] dcoarse sums of the other slot groups
  const long long block = blockIdx.x;
  for (int i = threadIdx.x; i < kBlock; i += blockDim.x) {
    const long long slot = block * kBlock + i;
    rows[i] = p.slot_row != nullptr ? p.slot_row[slot] : slot;
  }
  __syncthreads();
  const int width = p.heads * kDim;
  const int chunks = width / kChunk;
  const long long slots = p.blocks * kBlock;
  const int local = threadIdx.x % cols, group = threadIdx.x / cols;
  const int c = blockIdx.y * cols + local;
  // `cols` is a multiple of 16, so an aligned group of 16 lanes holds one head of one slot group.
  const bool active = c < chunks;
  const int head = active ? (c * kChunk) / kDim : 0;
  const int per = kBlock / groups;
  const long long coarse_row = (p.block_coarse != nullptr && p.coarse != nullptr) ? p.block_coarse[block] : -1;
  const uint4* grad = reinterpret_cast<const uint4*>(p.grad);
  const uint4* gate = reinterpret_cast<const uint4*>(p.gate);
  const uint4* fine = reinterpret_cast<const uint4*>(p.o_slots);
  float cz[8] = {};
  if (active && coarse_row >= 0) accumulate(cz, __ldg(reinterpret_cast<const uint4*>(p.coarse) + coarse_row * chunks + c));
  // gate and dgate rows may be strided (one field of an interleaved tensor): 16-byte units.
  const long long io_row = p.io_row_stride / kChunk;
  const long long io_col = (c / (kDim / kChunk)) * (p.io_head_stride / kChunk) + c % (kDim / kChunk);
  float dc[8] = {};
#pragma unroll 2
  for (int s = group * per; s < (group + 1) * per; ++s) {
    const long long row = rows[s];
    const long long slot = block * kBlock + s;
    float g[8] = {}, o[8] = {};
    uint4 gv = make_uint4(0, 0, 0, 0);
    if (active && row >= 0) {
      gv = __ldg(grad + row * chunks + c);
      const uint4 ov = __ldg(fine + slot * chunks + c);
      uint4 tv = make_uint4(0, 0, 0, 0);
      if (coarse_row >= 0) tv = __ldg(gate + row * io_row + io_col);
      accumulate(g, gv);
      accumulate(o, ov);
      if (coarse_row >= 0) {
        float gt[8] = {};
        accumulate(gt, tv);
        float dg[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          dg[e] = g[e] * cz[e];
          dc[e] += g[e] * gt[e];
        }
        if (p.dgate != nullptr)
          reinterpret_cast<uint4*>(p.dgate)[row * io_row + io_col] =
              make_uint4(pack_bf16(dg[0], dg[1]), pack_bf16(dg[2], dg[3]), pack_bf16(dg[4], dg[5]),
                         pack_bf16(dg[6], dg[7]));
      } else if (p.dgate != nullptr) {
        reinterpret_cast<uint4*>(p.dgate)[row * io_row + io_col] = make_uint4(0, 0, 0, 0);
      }
    }
    if (active && p.grad_slots != nullptr) reinterpret_cast<uint4*>(p.grad_slots)[slot * chunks + c] = gv;
    float part = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) part += g[e] * o[e];
    part = head_sum(part);
    if (active && (threadIdx.x & 15) == 0) p.delta[head * slots + slot] = part;
  }
  if (coarse_row < 0 || p.dcoarse == nullptr) return;  // uniform over the CTA
  if (groups > 1) {
    if (group > 0) {
      float* mine = partial + (static_cast<size_t>(group - 1) * cols + local) * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) mine[e] = dc[e];
    }
    __syncthreads();
    if (group > 0) return;
    for (int g2 = 1; g2 < groups; ++g2) {
      const float* other = partial + (static_cast<size_t>(g2 - 1) * cols + local) * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) dc[e] += other[e];
    }
  }
  const uint4 packed = make_uint4(pack_bf16(dc[0], dc[1]), pack_bf16(dc[2], dc[3]), pack_bf16(dc[4], dc[5]),
                                  pack_bf16(dc[6], dc[7]));
  if (active) reinterpret_cast<uint4*>(p.dcoarse)[coarse_row * chunks + c] = packed;
  float rounded[8] = {};
  accumulate(rounded, packed);
  float part = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) part += rounded[e] * cz[e];
  part = head_sum(part);
  if (active && p.coarse_delta != nullptr && (threadIdx.x & 15) == 0)
    p.coarse_delta[head * p.coarse_rows + coarse_row] = part;
}

// Ring epilogue of the forward pass: FP32 fine output in slot order -> BF16 copy for the backward
// pass and the merged result `fine + gate * coarse[block]` in the caller's row order.
__global__ void gate_merge_kernel(const float* __restrict__ fine, const int64_t* __restrict__ slot_row,
                                  const int32_t* __restrict__ block_coarse, const __nv_bfloat16* __restrict__ gate,
                                  const __nv_bfloat16* __restrict__ coarse, __nv_bfloat16* __restrict__ o_slots,
                                  __nv_bfloat16* __restrict__ out, int width, long long out_rows, int cols,
                                  int groups) {
  const long long block = blockIdx.x;
  const int chunks = width / kChunk;
  const long long coarse_row = (block_coarse != nullptr && coarse != nullptr) ? block_coarse[block] : -1;
  const int c = blockIdx.y * cols + threadIdx.x % cols, group = threadIdx.x / cols, per = kBlock / groups;
  if (c < chunks) {
    float cz[8] = {};
    if (coarse_row >= 0) accumulate(cz, __ldg(reinterpret_cast<const uint4*>(coarse) + coarse_row * chunks + c));
#pragma unroll 4
    for (int s = group * per; s < (group + 1) * per; ++s) {
      const long long slot = block * kBlock + s;
      const float4* src = reinterpret_cast<const float4*>(fine + slot * width + c * kChunk);
      const float4 a = src[0], b = src[1];
      float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      if (o_slots != nullptr)
        reinterpret_cast<uint4*>(o_slots)[slot * chunks + c] =
            make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
      const long long row = slot_row != nullptr ? slot_row[slot] : slot;
      if (row < 0 || row >= out_rows) continue;
      if (coarse_row >= 0) {
        float g[8] = {};
        accumulate(g, __ldg(reinterpret_cast<const uint4*>(gate) + row * chunks + c));
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = __fadd_rn(f[e], __fmul_rn(g[e], cz[e]));
      }
      reinterpret_cast<uint4*>(out)[row * chunks + c] =
          make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
    }
  }
}

// Ring epilogue of the backward pass: FP32 slot-order gradient + pooled-mean term -> BF16 rows.
__global__ void grad_finish_kernel(const float* __restrict__ acc, const int64_t* __restrict__ slot_row,
                                   const void* __restrict__ pool, int pool_f32, const int32_t* __restrict__ block_map,
                                   const int32_t* __restrict__ sizes, __nv_bfloat16* __restrict__ out, int width,
                                   long long out_rows, int cols, int groups) {
  const long long block = blockIdx.x;
  const int chunks = width / kChunk;
  long long prow = -1;
  if (pool != nullptr) prow = pool_f32 ? block : (block_map != nullptr ? block_map[block] : -1);
  const int size = sizes != nullptr ? sizes[block] : kBlock;
  const float inv = 1.f / static_cast<float>(size > 1 ? size : 1);
  const int c = blockIdx.y * cols + threadIdx.x % cols, group = threadIdx.x / cols, per = kBlock / groups;
  if (c < chunks) {
    float term[8] = {};
    if (prow >= 0) {
      if (pool_f32) {
        const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(pool) + prow * width + c * kChunk);
        const float4 a = src[0], b = src[1];
        term[0] = a.x, term[1] = a.y, term[2] = a.z, term[3] = a.w, term[4] = b.x, term[5] = b.y, term[6] = b.z,
        term[7] = b.w;
      } else {
        accumulate(term, __ldg(reinterpret_cast<const uint4*>(pool) + prow * chunks + c));
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) term[e] *= inv;
    }
#pragma unroll 4
    for (int s = group * per; s < (group + 1) * per; ++s) {
      const long long slot = block * kBlock + s;
      const long long row = slot_row != nullptr ? slot_row[slot] : slot;
      if (row < 0 || row >= out_rows) continue;
      const float4* src = reinterpret_cast<const float4*>(acc + slot * width + c * kChunk);
      const float4 a = src[0], b = src[1];
      const float f[8] = {a.x + term[0], a.y + term[1], a.z + term[2], a.w + term[3],
                          b.x + term[4], b.y + term[5], b.z + term[6], b.w + term[7]};
      reinterpret_cast<uint4*>(out)[row * chunks + c] =
          make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
    }
  }
}

}  // namespace

cudaError_t launch_slots_pool(const PoolParams& params, cudaStream_t stream) {
  if (params.blocks == 0) return cudaSuccess;
  const BlockShape shape = block_shape(params.width / kChunk);
  const size_t smem = static_cast<size_t>(shape.groups - 1) * shape.cols * 24 * sizeof(float);
  dim3 grid(static_cast<unsigned>(params.blocks), shape.parts);
  slots_pool_kernel<<<grid, shape.cols * shape.groups, smem, stream>>>(params, shape.cols, shape.groups);
  return cudaGetLastError();
}

cudaError_t launch_merge_bwd(const MergeBwdParams& params, cudaStream_t stream) {
  if (params.blocks == 0) return cudaSuccess;
  const BlockShape shape = block_shape(params.heads * kDim / kChunk);
  const size_t smem = static_cast<size_t>(shape.groups - 1) * shape.cols * 8 * sizeof(float);
  dim3 grid(static_cast<unsigned>(params.blocks), shape.parts);
  merge_bwd_kernel<<<grid, shape.cols * shape.groups, smem, stream>>>(params, shape.cols, shape.groups);
  return cudaGetLastError();
}

cudaError_t launch_gate_merge(const float* fine, const int64_t* slot_row, const int32_t* block_coarse,
                              const __nv_bfloat16* gate, const __nv_bfloat16* coarse, __nv_bfloat16* o_slots,
                              __nv_bfloat16* out, long long blocks, int heads, long long out_rows,
                              cudaStream_t stream) {
  if (blocks == 0) return cudaSuccess;
  const int width = heads * kDim;
  const BlockShape shape = block_shape(width / kChunk);
  gate_merge_kernel<<<dim3(static_cast<unsigned>(blocks), shape.parts), shape.cols * shape.groups, 0, stream>>>(
      fine, slot_row, block_coarse, gate, coarse, o_slots, out, width, out_rows, shape.cols, shape.groups);
  return cudaGetLastError();
}

cudaError_t launch_grad_finish(const float* acc, const int64_t* slot_row, const void* pool, int pool_f32,
                               const int32_t* block_map, const int32_t* sizes, __nv_bfloat16* out, long long blocks,
                               int heads, long long out_rows, cudaStream_t stream) {
  if (blocks == 0) return cudaSuccess;
  const int width = heads * kDim;
  const BlockShape shape = block_shape(width / kChunk);
  grad_finish_kernel<<<dim3(static_cast<unsigned>(blocks), shape.parts), shape.cols * shape.groups, 0, stream>>>(
      acc, slot_row, pool, pool_f32, block_map, sizes, out, width, out_rows, shape.cols, shape.groups);
  return cudaGetLastError();
}

}  // namespace vsa
