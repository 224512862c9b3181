// Block-sparse fine attention, forward, for sm_100a.
//
// One CTA owns one (query block, head): 64 query rows against the listed 64-slot KV blocks.
// K and V tiles arrive by TMA (128-byte swizzle), S = Q K^T and O += P V run on tcgen05 with
// the accumulators in tensor memory, the softmax runs on all 128 threads (two threads per
// query row, 32 score columns each) with the running maximum raised only when it grew by more
// than 2^8 (the accumulated O is rescaled in TMEM only then).  The epilogue writes the
// normalised fine output in slot order, the natural-log LSE, and - when a row map is given -
// the merged result `fine + gate * coarse[block]` straight into the caller's row order, which
// replaces the reference's separate restore and gate-add passes
// (reference vsa_core.py:15-20, vsa_kernels.py:191-201, vsa.py:111-117).
#include "vsa_common.cuh"
#include "vsa_kernels.h"

namespace vsa {

namespace {

constexpr int kThreads = 128;
constexpr int kTmemCols = 256;     // S0 [0,64)  S1 [64,128)  O [128,256)
constexpr uint32_t kColO = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct __align__(1024) FwdSmem {
  uint8_t q[kTileBytes];
  uint8_t k[2][kTileBytes];
  uint8_t v[2][kTileBytes];
  uint8_t p[kHalfTileBytes];
  uint64_t q_full, k_full[2], v_full[2], s_done[2], o_done;
  uint32_t tmem_base;
  int abort_flag;
};

VSA_DEVICE float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// S[buf] = Q K^T for the K tile in stage `stage`: eight K=16 steps over the two 64-wide halves.
VSA_DEVICE void issue_qk(uint32_t tmem_s, const uint8_t* q, const uint8_t* k) {
  constexpr uint32_t idesc = umma_idesc(64, 64, 0, 0);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const uint32_t off = (ks >> 2) * kHalfTileBytes + (ks & 3) * 32;
    umma_ss(tmem_s, umma_smem_desc(smem_u32(q) + off, 16, 1024), umma_smem_desc(smem_u32(k) + off, 16, 1024),
            idesc, ks > 0);
  }
}

// O (+)= P V: P is K-major [64 q][64 kv]; V is MN-major ([kv][d], two 64-wide d halves).
VSA_DEVICE void issue_pv(uint32_t tmem_o, const uint8_t* p, const uint8_t* v, bool accumulate) {
  constexpr uint32_t idesc = umma_idesc(64, 128, 0, 1);
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    umma_ss(tmem_o, umma_smem_desc(smem_u32(p) + ks * 32, 16, 1024),
            umma_smem_desc(smem_u32(v) + ks * 2048, kHalfTileBytes, 1024), idesc, accumulate || ks > 0);
  }
}

}  // namespace

template <bool kMerge>
__global__ void __launch_bounds__(kThreads) fine_fwd_kernel(const __grid_constant__ FineFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  FwdSmem& sm = *reinterpret_cast<FwdSmem*>(
      smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qb = blockIdx.x, head = blockIdx.y;
  const int row = warp * 16 + (lane & 15);  // query row inside the block
  const int half = lane >> 4;               // which 32 score columns / 64 output columns
  const int n = p.counts[static_cast<long long>(head) * p.count_head_stride + qb];
  const int32_t* list = p.indices + static_cast<long long>(head) * p.index_head_stride +
                        static_cast<long long>(qb) * p.capacity;

  if (tid == 0) {
    mbar_init(&sm.q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.k_full[i], 1);
      mbar_init(&sm.v_full[i], 1);
      mbar_init(&sm.s_done[i], 1);
    }
    mbar_init(&sm.o_done, 1);
    sm.abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&p.q_map);
    tma_prefetch_desc(&p.k_map);
    tma_prefetch_desc(&p.v_map);
  }
  if (warp == 0) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  volatile int* abort_flag = &sm.abort_flag;

  if (tid == 0 && n > 0) {
    mbar_expect_tx(&sm.q_full, kTileBytes);
    tma_load_tile(sm.q, &p.q_map, &sm.q_full, head, qb);
    for (int s = 0; s < 2 && s < n; ++s) {
      mbar_expect_tx(&sm.k_full[s], kTileBytes);
      tma_load_tile(sm.k[s], &p.k_map, &sm.k_full[s], head, list[s]);
      mbar_expect_tx(&sm.v_full[s], kTileBytes);
      tma_load_tile(sm.v[s], &p.v_map, &sm.v_full[s], head, list[s]);
    }
    mbar_wait(&sm.q_full, 0, abort_flag, p.status, 1);
    mbar_wait(&sm.k_full[0], 0, abort_flag, p.status, 2);
    tc_fence_after();
    issue_qk(tmem, sm.q, sm.k[0]);
    umma_commit(&sm.s_done[0]);
  }

  const float sl2 = p.scale * kLog2e;
  float m_ref = -INFINITY;  // running reference maximum of the raw scores
  float l = 0.f;            // running sum of exp2((s - m_ref) * sl2) over this thread's columns

  for (int j = 0; j < n; ++j) {
    const int b = j & 1;
    const uint32_t phase = (j >> 1) & 1;
    const int kv_block = list[j];
    const int kv_size = p.kv_sizes != nullptr ? p.kv_sizes[kv_block] : kBlock;

    mbar_wait(&sm.s_done[b], phase, abort_flag, p.status, 3);
    tc_fence_after();
    if (tid == 0) {
      // S_j is complete, so K stage b is free and S buffer b^1 was drained one iteration ago.
      if (j + 2 < n) {
        mbar_expect_tx(&sm.k_full[b], kTileBytes);
        tma_load_tile(sm.k[b], &p.k_map, &sm.k_full[b], head, list[j + 2]);
      }
      if (j + 1 < n) {
        mbar_wait(&sm.k_full[b ^ 1], ((j + 1) >> 1) & 1, abort_flag, p.status, 4);
        tc_fence_after();
        issue_qk(tmem + (b ^ 1) * 64, sm.q, sm.k[b ^ 1]);
        umma_commit(&sm.s_done[b ^ 1]);
      }
    }
    __syncwarp();
    uint32_t s_bits[32];
    VSA_TMEM_LD_16x32bx2_X32(s_bits, tmem + lane_base + b * 64, 32);
    tmem_wait_ld();

    float s[32];
    float m_tile = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      s[i] = (half * 32 + i < kv_size) ? __uint_as_float(s_bits[i]) : -INFINITY;
      m_tile = fmaxf(m_tile, s[i]);
    }
    m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 16));
    const float m_new = fmaxf(m_ref, m_tile);
    // Raise the reference maximum only when it moved by more than 2^8; both threads of a row
    // see the same m_tile, so they decide alike.
    const bool raise = (m_new > m_ref) && (m_ref == -INFINITY || (m_new - m_ref) * sl2 > kRescaleThreshold);
    float alpha = 1.f;
    if (raise) {
      alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2((m_ref - m_new) * sl2);
      m_ref = m_new;
    }
    const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref * sl2;
    float row_sum = 0.f;
    uint32_t packed[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      const float p0 = fast_exp2(s[i] * sl2 - m_use);
      const float p1 = fast_exp2(s[i + 1] * sl2 - m_use);
      packed[i >> 1] = pack_bf16(p0, p1);
      // Sum what the tensor core will see, so that l matches the BF16 P used for O.
      const float2 seen = unpack_bf16(packed[i >> 1]);
      row_sum += seen.x + seen.y;
    }
    l = l * alpha + row_sum;

    // PV_{j-1} must be finished before P is overwritten or O rescaled.
    if (j > 0) {
      mbar_wait(&sm.o_done, (j - 1) & 1, abort_flag, p.status, 5);
      tc_fence_after();
      if (tid == 0 && j + 1 < n && j + 1 >= 2) {
        // V stage (j+1)&1 was last read by PV_{j-1}.
        mbar_expect_tx(&sm.v_full[b ^ 1], kTileBytes);
        tma_load_tile(sm.v[b ^ 1], &p.v_map, &sm.v_full[b ^ 1], head, list[j + 1]);
      }
      __syncwarp();
      if (__any_sync(0xffffffffu, raise)) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t o_bits[32];
          const uint32_t addr = tmem + lane_base + kColO + c * 32;
          VSA_TMEM_LD_16x32bx2_X32(o_bits, addr, 64);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_bits[i] = __float_as_uint(__uint_as_float(o_bits[i]) * alpha);
          VSA_TMEM_ST_16x32bx2_X32(o_bits, addr, 64);
        }
        tmem_wait_st();
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint4 v4 = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      *reinterpret_cast<uint4*>(sm.p + swizzled_offset(row, half * 4 + c)) = v4;
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      mbar_wait(&sm.v_full[b], phase, abort_flag, p.status, 6);
      tc_fence_after();
      issue_pv(tmem + kColO, sm.p, sm.v[b], j > 0);
      umma_commit(&sm.o_done);
    }
  }

  // ---------------------------------------------------------------- epilogue
  float o[64];
  if (n > 0) {
    mbar_wait(&sm.o_done, (n - 1) & 1, abort_flag, p.status, 7);
    tc_fence_after();
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t o_bits[32];
      VSA_TMEM_LD_16x32bx2_X32(o_bits, tmem + lane_base + kColO + c * 32, 64);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) o[c * 32 + i] = __uint_as_float(o_bits[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 64; ++i) o[i] = 0.f;
  }
  l += __shfl_xor_sync(0xffffffffu, l, 16);
  const float inv = l > 0.f ? 1.f / l : 0.f;
  const float lse = l > 0.f ? m_ref * p.scale + logf(l) : -INFINITY;
  const long long slot = static_cast<long long>(qb) * kBlock + row;
  const long long width = static_cast<long long>(p.heads) * kDim;
  const long long col = static_cast<long long>(head) * kDim + half * 64;
  if (half == 0) p.lse[static_cast<long long>(head) * p.q_slots + slot] = lse;
#pragma unroll
  for (int i = 0; i < 64; ++i) o[i] *= inv;
  {
    uint4* dst = reinterpret_cast<uint4*>(p.o_slots + slot * width + col);
#pragma unroll
    for (int c = 0; c < 8; ++c)
      dst[c] = make_uint4(pack_bf16(o[8 * c], o[8 * c + 1]), pack_bf16(o[8 * c + 2], o[8 * c + 3]),
                          pack_bf16(o[8 * c + 4], o[8 * c + 5]), pack_bf16(o[8 * c + 6], o[8 * c + 7]));
  }
  if (kMerge) {
    const long long out_row = p.slot_row != nullptr ? p.slot_row[slot] : slot;
    if (out_row >= 0 && out_row < p.out_rows) {
      const int coarse_slot = p.block_coarse != nullptr ? p.block_coarse[qb] : -1;
      uint4* dst = reinterpret_cast<uint4*>(p.out + out_row * width + col);
      if (coarse_slot >= 0) {
        const uint4* gate = reinterpret_cast<const uint4*>(p.gate + out_row * width + col);
        const uint4* coarse = reinterpret_cast<const uint4*>(p.coarse + coarse_slot * width + col);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 g = gate[c], cz = __ldg(coarse + c);
          const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, cw[4] = {cz.x, cz.y, cz.z, cz.w};
          uint32_t r[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 gf = unpack_bf16(gw[e]), cf = unpack_bf16(cw[e]);
            // Product and sum are rounded separately, as the reference's merge does.
            r[e] = pack_bf16(__fadd_rn(o[8 * c + 2 * e], __fmul_rn(gf.x, cf.x)),
                             __fadd_rn(o[8 * c + 2 * e + 1], __fmul_rn(gf.y, cf.y)));
          }
          dst[c] = make_uint4(r[0], r[1], r[2], r[3]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c)
          dst[c] = make_uint4(pack_bf16(o[8 * c], o[8 * c + 1]), pack_bf16(o[8 * c + 2], o[8 * c + 3]),
                              pack_bf16(o[8 * c + 4], o[8 * c + 5]), pack_bf16(o[8 * c + 6], o[8 * c + 7]));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

size_t fine_fwd_smem_bytes() { return sizeof(FwdSmem) + 1024; }

cudaError_t launch_fine_fwd(const FineFwdParams& params, bool merge, cudaStream_t stream) {
  const size_t smem = fine_fwd_smem_bytes();
  auto kernel = merge ? fine_fwd_kernel<true> : fine_fwd_kernel<false>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (err != cudaSuccess) return err;
  dim3 grid(params.q_blocks, params.heads);
  kernel<<<grid, kThreads, smem, stream>>>(params);
  return cudaGetLastError();
}

}  // namespace vsa
