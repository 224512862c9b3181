// Block-sparse fine attention, forward, for sm_100a.
//
// One CTA owns one (query block, head): 64 query rows against the listed 64-slot KV blocks.
// K and V tiles arrive by TMA (128-byte swizzle).  Two tcgen05 products per tile:
//   S   = Q K^T          M = 64 query rows,  N = 64 keys,    K = 128   (accumulator: 64 columns)
//   O^T += V^T P^T       M = 128 head dims,  N = 64 queries, K = 64    (accumulator: 64 columns)
// The output is kept transposed so that its product runs with M = 128, the shape at which the
// tensor core works at full rate (M = 64 uses half of its lanes).  V is read as an MN-major A
// operand and P, written row-major [query][key] by the softmax threads, is the K-major B
// operand, so nothing is transposed in shared memory.  The softmax runs on all 128 threads (two
// threads per query row, 32 score columns each); the running maximum is raised only when it grew
// by more than 2^8, and only then is O^T rescaled in tensor memory.  Two more warps run ahead of
// the softmax: one issues the TMA loads, one the MMAs.  S is double-buffered in tensor memory and
// K, V and P have two shared-memory stages each, so S_{j+1} is ready before the softmax of tile j
// ends, the softmax of tile j+1 does not wait for the P V product of tile j, and the next tiles
// are fetched under the current one.  Two CTAs share an SM.  The epilogue writes the normalised fine output in slot order, the natural-log
// LSE and - when a row map is given - the merged result `fine + gate * coarse[block]` straight
// into the caller's row order, which replaces the reference's separate restore and gate-add
// passes (reference vsa_core.py:15-20, vsa_kernels.py:191-201, vsa.py:111-117).
#include "vsa_common.cuh"
#include "vsa_kernels.h"

namespace vsa {

namespace {

constexpr int kSoftmaxThreads = 128;  // warps 0..3: softmax and epilogue
constexpr int kThreads = 192;         // warp 4: tcgen05.mma issue, warp 5: TMA loads
constexpr int kTmemCols = 256;        // S0 [0,64)  S1 [64,128)  O^T [128,192)
constexpr uint32_t kColO = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct FwdSmem {  // placed at a 1024-byte aligned address; every tile offset is a multiple of 1024
  uint8_t q[kTileBytes];
  uint8_t k[2][kTileBytes];
  uint8_t v[2][kTileBytes];
  uint8_t p[2][kHalfTileBytes];
  float alpha[2][kBlock];   // per tile of the pair and query row: factor applied when the maximum is raised
  float inv_l[kBlock];      // per query row: 1 / softmax denominator (epilogue)
  long long out_row[kBlock];
  uint64_t q_full, k_full[2], v_full[2], s_done, o_done, s_free, p_ready;
  uint32_t tmem_base;
  int abort_flag;
};

VSA_DEVICE float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// S = Q K^T: eight K=16 steps over the two 64-wide halves of the head dimension.
VSA_DEVICE void issue_qk(uint32_t tmem_s, const uint8_t* q, const uint8_t* k) {
  constexpr uint32_t idesc = umma_idesc(64, 64, 0, 0);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const uint32_t off = (ks >> 2) * kHalfTileBytes + (ks & 3) * 32;
    umma_ss(tmem_s, umma_smem_desc(smem_u32(q) + off, 16, 1024), umma_smem_desc(smem_u32(k) + off, 16, 1024),
            idesc, ks > 0);
  }
}

// O^T (+)= V^T P^T.  A = V tile [key][dim] read MN-major (two 64-wide dim halves 8 KiB apart,
// 16 keys = 2 KiB per K step); B = P [query][key], K-major (32 bytes per K step).
VSA_DEVICE void issue_pv(uint32_t tmem_o, const uint8_t* p, const uint8_t* v, bool accumulate) {
  constexpr uint32_t idesc = umma_idesc(128, 64, 1, 0);
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    umma_ss(tmem_o, umma_smem_desc(smem_u32(v) + ks * 2048, kHalfTileBytes, 1024),
            umma_smem_desc(smem_u32(p) + ks * 32, 16, 1024), idesc, accumulate || ks > 0);
  }
}

}  // namespace

template <bool kMerge>
__global__ void __launch_bounds__(kThreads, 2) fine_fwd_kernel(const __grid_constant__ FineFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  FwdSmem& sm = *reinterpret_cast<FwdSmem*>(smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qb = blockIdx.x, head = blockIdx.y;
  const int row = warp * 16 + (lane & 15);  // query row inside the block (softmax role)
  const int half = lane >> 4;               // which 32 score columns
  const int n = p.counts[static_cast<long long>(head) * p.count_head_stride + qb];
  const int32_t* list = p.indices + static_cast<long long>(head) * p.index_head_stride +
                        static_cast<long long>(qb) * p.capacity;

  if (tid == 0) {
    mbar_init(&sm.q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.k_full[i], 1);
      mbar_init(&sm.v_full[i], 1);
    }
    mbar_init(&sm.s_done, 1);
    mbar_init(&sm.o_done, 1);
    mbar_init(&sm.s_free, kSoftmaxThreads);
    mbar_init(&sm.p_ready, kSoftmaxThreads);
    sm.abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&p.q_map);
    tma_prefetch_desc(&p.k_map);
    tma_prefetch_desc(&p.v_map);
  }
  if (kMerge && tid < kBlock) {
    const long long slot = static_cast<long long>(qb) * kBlock + tid;
    sm.out_row[tid] = p.slot_row != nullptr ? p.slot_row[slot] : slot;
  }
  if (warp == 0) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  volatile int* abort_flag = &sm.abort_flag;

  const float sl2 = p.scale * kLog2e;
  float m_ref = -INFINITY;  // running reference maximum of the raw scores
  float l = 0.f;            // running sum of exp2((s - m_ref) * sl2) over this thread's columns

  // Tiles are processed two at a time ("pair" i = tiles 2i and 2i+1): the softmax warps pull both
  // score tiles into registers, release the S buffers, and pay for one fence, one consensus
  // barrier and one arrival per pair.  Barrier discipline: a barrier is only ever waited on for its
  // NEWEST commit or arrival round (a wait for an older phase could find the barrier two phases
  // ahead and block); every producer/consumer edge below is ordered so that this holds.
  const int pairs = (n + 1) >> 1;
  if (warp == 5) {
    // ------------------------------------------------------------ producer: TMA loads
    if (lane == 0 && n > 0) {
      mbar_expect_tx(&sm.q_full, kTileBytes);
      tma_load_tile(sm.q, &p.q_map, &sm.q_full, head, qb);
      auto load_k = [&](int i) {
        for (int t = 0; t < 2 && 2 * i + t < n; ++t) {
          mbar_expect_tx(&sm.k_full[t], kTileBytes);
          tma_load_tile(sm.k[t], &p.k_map, &sm.k_full[t], head, list[2 * i + t]);
        }
      };
      load_k(0);
      for (int i = 0; i < pairs; ++i) {
        // The S products of pair i finish before the P V products of pair i-1 (they are issued
        // first), so K of pair i+1 is fetched before V of pair i: each load starts as soon as its
        // stage is free.  Both waits are for the newest commit on their barrier (pair i+1 cannot
        // be issued before these loads land).
        if (i + 1 < pairs) {
          mbar_wait(&sm.s_done, i & 1, abort_flag, p.status, 3);
          load_k(i + 1);
        }
        if (i > 0) mbar_wait(&sm.o_done, (i - 1) & 1, abort_flag, p.status, 10);
        for (int t = 0; t < 2 && 2 * i + t < n; ++t) {
          mbar_expect_tx(&sm.v_full[t], kTileBytes);
          tma_load_tile(sm.v[t], &p.v_map, &sm.v_full[t], head, list[2 * i + t]);
        }
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------ issuer: MMAs
    if (lane == 0 && n > 0) {
      mbar_wait(&sm.q_full, 0, abort_flag, p.status, 1);
      for (int i = 0; i < pairs; ++i) {
        const int count = (2 * i + 1 < n) ? 2 : 1;
        // S buffers are free once every softmax thread holds pair i-1 in registers.
        if (i > 0) mbar_wait(&sm.s_free, (i - 1) & 1, abort_flag, p.status, 8);
        for (int t = 0; t < count; ++t) {
          mbar_wait(&sm.k_full[t], i & 1, abort_flag, p.status, 2);
          tc_fence_after();
          issue_qk(tmem + t * 64, sm.q, sm.k[t]);
        }
        umma_commit(&sm.s_done);
        if (i > 0) {
          // P of pair i-1 is written; its P V products follow the S products of pair i so that
          // the next softmax never waits for them.
          const int prev = (2 * i - 1 < n) ? 2 : 1;
          mbar_wait(&sm.p_ready, (i - 1) & 1, abort_flag, p.status, 9);
          for (int t = 0; t < prev; ++t) {
            mbar_wait(&sm.v_full[t], (i - 1) & 1, abort_flag, p.status, 6);
            tc_fence_after();
            issue_pv(tmem + kColO, sm.p[t], sm.v[t], i > 1 || t > 0);
          }
          umma_commit(&sm.o_done);
        }
      }
      const int last = pairs - 1, count = (2 * last + 1 < n) ? 2 : 1;
      mbar_wait(&sm.p_ready, last & 1, abort_flag, p.status, 9);
      for (int t = 0; t < count; ++t) {
        mbar_wait(&sm.v_full[t], last & 1, abort_flag, p.status, 6);
        tc_fence_after();
        issue_pv(tmem + kColO, sm.p[t], sm.v[t], last > 0 || t > 0);
      }
      umma_commit(&sm.o_done);
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    // The valid length of a tile comes from two dependent global loads (list, then sizes); they
    // are issued one pair ahead so their latency never sits in the loop.
    int size_next[2] = {kBlock, kBlock};
    if (p.kv_sizes != nullptr) {
      if (n > 0) size_next[0] = p.kv_sizes[list[0]];
      if (n > 1) size_next[1] = p.kv_sizes[list[1]];
    }
    for (int i = 0; i < pairs; ++i) {
      const int count = (2 * i + 1 < n) ? 2 : 1;
      const int kv_size[2] = {size_next[0], size_next[1]};
      if (p.kv_sizes != nullptr) {
        if (2 * i + 2 < n) size_next[0] = p.kv_sizes[list[2 * i + 2]];
        if (2 * i + 3 < n) size_next[1] = p.kv_sizes[list[2 * i + 3]];
      }
      mbar_wait(&sm.s_done, i & 1, abort_flag, p.status, 3);
      tc_fence_after();
      uint32_t s_bits[2][32];
      VSA_TMEM_LD_16x32bx2_X32(s_bits[0], tmem + lane_base, 32);
      if (count == 2) VSA_TMEM_LD_16x32bx2_X32(s_bits[1], tmem + lane_base + 64, 32);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&sm.s_free);

      bool raise_any = false;
      uint32_t packed[2][16];
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (t < count) {
          float s[32];
          if (kv_size[t] < kBlock) {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              s[e] = (half * 32 + e < kv_size[t]) ? __uint_as_float(s_bits[t][e]) : -INFINITY;
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) s[e] = __uint_as_float(s_bits[t][e]);
          }
          // Four independent chains keep the dependent-latency path short.
          float m4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
          for (int e = 4; e < 32; ++e) m4[e & 3] = fmaxf(m4[e & 3], s[e]);
          float m_tile = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
          m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 16));
          const float m_new = fmaxf(m_ref, m_tile);
          // Raise the reference maximum only when it moved by more than 2^8; both threads of a
          // row see the same m_tile, so they decide alike.
          const bool raise = (m_new > m_ref) && (m_ref == -INFINITY || (m_new - m_ref) * sl2 > kRescaleThreshold);
          float alpha = 1.f;
          if (raise) {
            alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2((m_ref - m_new) * sl2);
            m_ref = m_new;
          }
          // alpha[t][row]: factor for everything accumulated before tile t of this pair.
          if (half == 0) sm.alpha[t][row] = alpha;
          raise_any |= raise && (i > 0 || t > 0);
          if (t == 1 && raise) {
            // Tile 0 of this pair was scaled with the old reference: bring its P up to date.
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const float2 f = unpack_bf16(packed[0][e]);
              packed[0][e] = pack_bf16(f.x * alpha, f.y * alpha);
            }
          }
          const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref * sl2;
          float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float p0 = fast_exp2(fmaf(s[e], sl2, -m_use));
            const float p1 = fast_exp2(fmaf(s[e + 1], sl2, -m_use));
            packed[t][e >> 1] = pack_bf16(p0, p1);
            sum4[(e >> 1) & 3] += p0 + p1;
          }
          l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        } else if (half == 0) {
          sm.alpha[t][row] = 1.f;
        }
      }
      // P buffers were last read by the P V products of pair i-1, the newest commit on o_done.
      if (i > 0) mbar_wait(&sm.o_done, (i - 1) & 1, abort_flag, p.status, 5);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (t < count) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(sm.p[t] + swizzled_offset(row, half * 4 + c)) =
                make_uint4(packed[t][4 * c], packed[t][4 * c + 1], packed[t][4 * c + 2], packed[t][4 * c + 3]);
        }
      }
      fence_proxy_async_smem();
      if (named_barrier_or(1, kSoftmaxThreads, raise_any)) {
        // Rare: scale column r of O^T (lane = head dim, column = query row) by the factors of
        // both tiles.  O^T is stable here: the P V products of pair i-1 are complete.
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t o_bits[32];
          const uint32_t addr = tmem + lane_base + kColO + c * 32;
          VSA_TMEM_LD_32x32b_X32(o_bits, addr);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e)
            o_bits[e] = __float_as_uint(__uint_as_float(o_bits[e]) * (sm.alpha[0][c * 32 + e] * sm.alpha[1][c * 32 + e]));
          VSA_TMEM_ST_32x32b_X32(o_bits, addr);
        }
        tmem_wait_st();
        // alpha[] is rewritten next iteration: every reader must be done first.
        named_barrier(1, kSoftmaxThreads);
      }
      tc_fence_before();
      mbar_arrive(&sm.p_ready);
    }
  }

  // ---------------------------------------------------------------- epilogue
  const long long width = static_cast<long long>(p.heads) * kDim;
  if (warp < 4) {
  l += __shfl_xor_sync(0xffffffffu, l, 16);
  if (half == 0) {
    sm.inv_l[row] = l > 0.f ? 1.f / l : 0.f;
    const long long slot = static_cast<long long>(qb) * kBlock + row;
    p.lse[static_cast<long long>(head) * p.q_slots + slot] = l > 0.f ? m_ref * p.scale + logf(l) : -INFINITY;
  }
  if (n > 0) {
    mbar_wait(&sm.o_done, (pairs - 1) & 1, abort_flag, p.status, 7);
    tc_fence_after();
  }
  named_barrier(1, kSoftmaxThreads);
  // Thread = head dim `dim`; its 64 accumulator columns are the 64 query rows.  A warp writes 32
  // consecutive BF16 (64 bytes) of one row per store.
  const int dim = tid;
  const long long col = static_cast<long long>(head) * kDim + dim;
  float coarse = 0.f;
  bool gated = false;
  if (kMerge) {
    const int coarse_slot = p.block_coarse != nullptr ? p.block_coarse[qb] : -1;
    gated = coarse_slot >= 0;
    if (gated) coarse = __bfloat162float(p.coarse[coarse_slot * width + col]);
  }
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t o_bits[32] = {};
    if (n > 0) {
      VSA_TMEM_LD_32x32b_X32(o_bits, tmem + lane_base + kColO + c * 32);
      tmem_wait_ld();
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int r = c * 32 + i;
      const float o = __uint_as_float(o_bits[i]) * sm.inv_l[r];
      const long long slot = static_cast<long long>(qb) * kBlock + r;
      p.o_slots[slot * width + col] = __float2bfloat16(o);
      if (kMerge) {
        const long long out_row = sm.out_row[r];
        if (out_row >= 0 && out_row < p.out_rows) {
          float merged = o;
          // Product and sum are rounded separately, as the reference's merge does.
          if (gated) merged = __fadd_rn(o, __fmul_rn(__bfloat162float(p.gate[out_row * width + col]), coarse));
          p.out[out_row * width + col] = __float2bfloat16(merged);
        }
      }
    }
  }
  }  // softmax warps
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
