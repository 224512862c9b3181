// Block-sparse fine attention, backward, for sm_100a: two tcgen05 kernels without atomics.
//
//   dQ kernel   one CTA per (query block, head), walks the block's KV list like the forward:
//               S = Q K^T, dP = dO V^T, dS = P * (dP - delta) * scale, dQ^T += K^T dS^T.
//   dK/dV kernel one CTA per (KV block, head), walks the query blocks that list this KV block
//               (a per-call bitmask built by build_kv_mask_kernel):
//               S = Q K^T, dP = dO V^T (query rows on the lanes, as in the dQ kernel, so each
//               thread needs one LSE and one delta), dV^T += dO^T P, dK^T += Q^T dS.
//
// The 64 x 64 score products run with M = 64; the three "x 128-wide" gradient products are kept
// transposed (head dim on the M axis) so that they run with M = 128, the tensor core's full-rate
// shape, and each accumulator needs only 64 TMEM columns: two CTAs fit on an SM.  P is
// recomputed from the saved LSE (natural log), so no softmax state is carried.  The epilogues
// add the gradient that reaches a row through its block's pooled mean and scatter the rows
// straight to the caller's row order, skipping padding slots.  Together they replace
// the reference's fine backward call and its slot-to-row gathers
// (reference vsa_core.py:23-30, 42-47; vsa_kernels.py:86-96, 161-176 adjoint).
#include "vsa_common.cuh"
#include "vsa_kernels.h"

namespace vsa {

namespace {

constexpr int kSoftmaxThreads = 128;  // warps 0..3: score math and epilogue
constexpr int kThreads = 160;         // warp 4: TMA and tcgen05.mma issue
constexpr float kLog2e = 1.4426950408889634f;

VSA_DEVICE float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The issue helpers build each operand's descriptor low word once per product and advance it
// with immediates: the issuing thread is alone in its warp, and per-MMA descriptor arithmetic
// would cost more cycles than the MMA runs for.
//
// D[64 x 64] = A[64 x 128] B[64 x 128]^T, both K-major tiles made of two 64-wide halves.
VSA_DEVICE void issue_nt_128(uint32_t tmem_d, const uint8_t* a, const uint8_t* b) {
  constexpr uint32_t idesc = umma_idesc(64, 64, 0, 0);
  const uint32_t a_lo = umma_desc_lo(smem_u32(a), 16), b_lo = umma_desc_lo(smem_u32(b), 16);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const uint32_t off = ((ks >> 2) * kHalfTileBytes + (ks & 3) * 32) >> 4;
    umma_ss_lo(tmem_d, a_lo + off, b_lo + off, idesc, ks > 0);
  }
}

// D^T[128 x 64] (+)= A^T B with A a row-major [64 rows][128 dims] tile read MN-major (M = dims,
// K = its rows) and B a K-major [64 rows][64] tile whose rows are the N index: the M = 128 form of
// the "x 128-wide output" products (dQ^T = K^T dS^T, dV^T = dO^T P, dK^T = Q^T dS).
VSA_DEVICE void issue_tn_128(uint32_t tmem_d, const uint8_t* a, const uint8_t* b, bool accumulate) {
  constexpr uint32_t idesc = umma_idesc(128, 64, 1, 0);
  const uint32_t a_lo = umma_desc_lo(smem_u32(a), kHalfTileBytes), b_lo = umma_desc_lo(smem_u32(b), 16);
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
    umma_ss_lo(tmem_d, a_lo + ks * (2048 >> 4), b_lo + ks * (32 >> 4), idesc, accumulate || ks > 0);
}

// D^T[128 x 64] (+)= A^T B with A a row-major [64 rows][128 dims] tile read MN-major and B a
// row-major [64 rows][64] BF16 tile read MN-major as well (rows of both are the K index):
// dV^T = dO^T P and dK^T = Q^T dS with P, dS stored [query][key].
VSA_DEVICE void issue_tt_128(uint32_t tmem_d, const uint8_t* a, const uint8_t* b, bool accumulate) {
  constexpr uint32_t idesc = umma_idesc(128, 64, 1, 1);
  const uint32_t a_lo = umma_desc_lo(smem_u32(a), kHalfTileBytes), b_lo = umma_desc_lo(smem_u32(b), kHalfTileBytes);
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
    umma_ss_lo(tmem_d, a_lo + ks * (2048 >> 4), b_lo + ks * (2048 >> 4), idesc, accumulate || ks > 0);
}

// Pooled-mean gradient of `block` at column `col`, already divided by the block size.
VSA_DEVICE float pool_term(const void* pool, int pool_f32, const int32_t* block_coarse, int block, int size,
                           long long width, long long col) {
  long long prow = -1;
  if (pool != nullptr) prow = pool_f32 ? block : (block_coarse != nullptr ? block_coarse[block] : -1);
  if (prow < 0) return 0.f;
  const float inv = 1.f / static_cast<float>(size > 1 ? size : 1);
  const float value = pool_f32 ? static_cast<const float*>(pool)[prow * width + col]
                               : __bfloat162float(static_cast<const __nv_bfloat16*>(pool)[prow * width + col]);
  return value * inv;
}

// Epilogue of a transposed accumulator: this thread owns head dim `col % 128`, its 64 columns are
// the 64 slots of `block`.  Adds `term` and writes BF16 to the mapped rows of `out`, or FP32 in
// slot order (added to the buffer's content when `accumulate`).  A warp store covers 32
// consecutive elements of one row.
VSA_DEVICE void store_grad_columns(bool have_acc, uint32_t tmem_addr, float term, const long long* out_rows,
                                   long long out_limit, __nv_bfloat16* out, float* out_f32, bool accumulate,
                                   long long block, long long width, long long col) {
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t bits[32] = {};
    if (have_acc) {
      VSA_TMEM_LD_32x32b_X32(bits, tmem_addr + c * 32);
      tmem_wait_ld();
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int r = c * 32 + i;
      const float value = __uint_as_float(bits[i]) + term;
      if (out_f32 != nullptr) {
        float* dst = out_f32 + (block * kBlock + r) * width + col;
        *dst = accumulate ? *dst + value : value;
      } else {
        const long long row = out_rows[r];
        if (row >= 0 && row < out_limit) out[row * width + col] = __float2bfloat16(value);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ dQ
constexpr int kDqTmemCols = 256;  // S [0,64)  dP [64,128)  dQ^T [128,192)

struct DqSmem {  // placed at a 1024-byte aligned address
  uint8_t q[kTileBytes];
  uint8_t d_o[kTileBytes];
  uint8_t k[2][kTileBytes];
  uint8_t v[2][kTileBytes];
  uint8_t ds[kHalfTileBytes];
  long long out_row[kBlock];
  uint64_t qdo_full, kv_full[2], sp_done, dq_done, sp_free, ds_ready;
  uint32_t tmem_base;
  int abort_flag;
};

}  // namespace

__global__ void __launch_bounds__(kThreads, 2) fine_bwd_dq_kernel(const __grid_constant__ FineBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  DqSmem& sm = *reinterpret_cast<DqSmem*>(smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qb = blockIdx.x, head = blockIdx.y;
  const int row = (warp & 3) * 16 + (lane & 15);
  const int half = lane >> 4;
  const int n = p.counts[static_cast<long long>(head) * p.count_head_stride + qb];
  const int32_t* list = p.indices + static_cast<long long>(head) * p.index_head_stride +
                        static_cast<long long>(qb) * p.capacity;

  if (tid == 0) {
    mbar_init(&sm.qdo_full, 1);
    mbar_init(&sm.kv_full[0], 1);
    mbar_init(&sm.kv_full[1], 1);
    mbar_init(&sm.sp_done, 1);
    mbar_init(&sm.dq_done, 1);
    mbar_init(&sm.sp_free, kSoftmaxThreads);
    mbar_init(&sm.ds_ready, kSoftmaxThreads);
    sm.abort_flag = 0;
    fence_barrier_init();
  }
  if (tid < kBlock) {
    const long long s = static_cast<long long>(qb) * kBlock + tid;
    sm.out_row[tid] = p.q_slot_row != nullptr ? p.q_slot_row[s] : s;
  }
  if (warp == 0) {
    tmem_alloc(&sm.tmem_base, kDqTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  volatile int* abort_flag = &sm.abort_flag;

  if (warp == 4) {
    // ------------------------------------------------------------ issuer: TMA loads and MMAs
    if (lane == 0 && n > 0) {
      mbar_expect_tx(&sm.qdo_full, 2 * kTileBytes);
      tma_load_tile(sm.q, &p.q_map, &sm.qdo_full, head, qb);
      tma_load_tile(sm.d_o, &p.do_map, &sm.qdo_full, head, qb);
      for (int s = 0; s < 2 && s < n; ++s) {
        mbar_expect_tx(&sm.kv_full[s], 2 * kTileBytes);
        tma_load_tile(sm.k[s], &p.k_map, &sm.kv_full[s], head, list[s]);
        tma_load_tile(sm.v[s], &p.v_map, &sm.kv_full[s], head, list[s]);
      }
      mbar_wait(&sm.qdo_full, 0, abort_flag, p.status, 11);
      mbar_wait(&sm.kv_full[0], 0, abort_flag, p.status, 12);
      tc_fence_after();
      issue_nt_128(tmem, sm.q, sm.k[0]);
      issue_nt_128(tmem + 64, sm.d_o, sm.v[0]);
      umma_commit(&sm.sp_done);
      for (int j = 0; j < n; ++j) {
        const int b = j & 1;
        if (j + 1 < n) {
          // S_j and dP_j are in registers: the next pair may overwrite them and runs under the
          // score math of tile j.
          mbar_wait(&sm.sp_free, j & 1, abort_flag, p.status, 17);
          mbar_wait(&sm.kv_full[b ^ 1], ((j + 1) >> 1) & 1, abort_flag, p.status, 15);
          tc_fence_after();
          issue_nt_128(tmem, sm.q, sm.k[b ^ 1]);
          issue_nt_128(tmem + 64, sm.d_o, sm.v[b ^ 1]);
          umma_commit(&sm.sp_done);
        }
        mbar_wait(&sm.ds_ready, j & 1, abort_flag, p.status, 18);
        tc_fence_after();
        issue_tn_128(tmem + 128, sm.k[b], sm.ds, j > 0);  // dQ^T += K^T dS^T
        umma_commit(&sm.dq_done);
        if (j + 2 < n) {
          // Stage b is free once dQ_j (the newest commit on this barrier) has read K_j.
          mbar_wait(&sm.dq_done, j & 1, abort_flag, p.status, 14);
          mbar_expect_tx(&sm.kv_full[b], 2 * kTileBytes);
          tma_load_tile(sm.k[b], &p.k_map, &sm.kv_full[b], head, list[j + 2]);
          tma_load_tile(sm.v[b], &p.v_map, &sm.kv_full[b], head, list[j + 2]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ score math warps
    const long long slot = static_cast<long long>(qb) * kBlock + row;
    const float lse = p.lse[static_cast<long long>(head) * p.q_slots + slot];
    const float delta = p.delta[static_cast<long long>(head) * p.q_slots + slot];
    const float sl2 = p.scale * kLog2e;
    const float lse2 = lse * kLog2e;
    const bool row_live = lse != -INFINITY;
    for (int j = 0; j < n; ++j) {
      const int kv_block = list[j];
      const int kv_size = p.kv_sizes != nullptr ? p.kv_sizes[kv_block] : kBlock;
      mbar_wait(&sm.sp_done, j & 1, abort_flag, p.status, 13);
      tc_fence_after();
      uint32_t s_bits[32], dp_bits[32];
      VSA_TMEM_LD_16x32bx2_X32(s_bits, tmem + lane_base, 32);
      VSA_TMEM_LD_16x32bx2_X32(dp_bits, tmem + lane_base + 64, 32);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&sm.sp_free);
      uint32_t packed[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float ds[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const bool live = row_live && (half * 32 + i + e < kv_size);
          const float pr = live ? fast_exp2(fmaf(__uint_as_float(s_bits[i + e]), sl2, -lse2)) : 0.f;
          ds[e] = pr * (__uint_as_float(dp_bits[i + e]) - delta) * p.scale;
        }
        packed[i >> 1] = pack_bf16(ds[0], ds[1]);
      }
      if (j > 0) {
        // dQ_{j-1} has finished reading the dS buffer.
        mbar_wait(&sm.dq_done, (j - 1) & 1, abort_flag, p.status, 14);
      }
#pragma unroll
      for (int c = 0; c < 4; ++c)
        *reinterpret_cast<uint4*>(sm.ds + swizzled_offset(row, half * 4 + c)) =
            make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      fence_proxy_async_smem();
      mbar_arrive(&sm.ds_ready);
    }
    if (n > 0) {
      mbar_wait(&sm.dq_done, (n - 1) & 1, abort_flag, p.status, 16);
      tc_fence_after();
    }
    const long long width = static_cast<long long>(p.heads) * kDim;
    const long long col = static_cast<long long>(head) * kDim + tid;
    const int q_size = p.q_sizes != nullptr ? p.q_sizes[qb] : kBlock;
    const float term = pool_term(p.dq_pool, p.pool_f32, p.q_block_coarse, qb, q_size, width, col);
    store_grad_columns(n > 0, tmem + lane_base + 128, term, sm.out_row, p.q_out_rows, p.dq, p.dq_f32,
                       p.f32_accumulate != 0, qb, width, col);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kDqTmemCols);
}

// ------------------------------------------------------------------------------------------ dK, dV
namespace {

constexpr int kDkvTmemCols = 256;  // S^T [0,64)  dP^T [64,128)  dK^T [128,192)  dV^T [192,256)

// Exactly 112 KiB of tiles plus the barriers: two CTAs fit on an SM only without an alignment
// pad, so the kernel requires (and checks) a 1024-byte aligned dynamic shared memory base.
struct DkvSmem {
  uint8_t k[kTileBytes];
  uint8_t v[kTileBytes];
  uint8_t q[2][kTileBytes];
  uint8_t d_o[2][kTileBytes];
  uint8_t pt[kHalfTileBytes];
  uint8_t dst[kHalfTileBytes];
  long long out_row[kBlock];
  uint64_t kv_full, qd_full[2], sp_done, dkv_done, sp_free, pd_ready;
  uint32_t tmem_base;
  int abort_flag;
};

// Walks the set bits of one (head, KV block) row of the query-block bitmask in ascending order.
// Every thread that needs the sequence keeps its own cursor, so nothing is passed through
// shared memory.
struct MaskCursor {
  const uint32_t* words;
  int count, word;
  uint32_t bits;
  VSA_DEVICE MaskCursor(const uint32_t* w, int c) : words(w), count(c), word(0), bits(c > 0 ? w[0] : 0u) {}
  VSA_DEVICE int next() {
    while (bits == 0) {
      if (++word >= count) return 0;
      bits = words[word];
    }
    const int bit = __ffs(bits) - 1;
    bits &= bits - 1;
    return word * 32 + bit;
  }
};

}  // namespace

__global__ void __launch_bounds__(kThreads, 2) fine_bwd_dkv_kernel(const __grid_constant__ FineBwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  DkvSmem& sm = *reinterpret_cast<DkvSmem*>(smem_raw);
  if ((smem_u32(smem_raw) & 1023) != 0) {
    // The swizzled tiles need 1024-byte alignment; report instead of computing garbage.
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, kDevWaitTimeout + 99);
    return;
  }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvb = blockIdx.x, head = blockIdx.y;
  const int row = (warp & 3) * 16 + (lane & 15);  // query row inside the current block (score math role)
  const int half = lane >> 4;                     // which 32 key columns
  const uint32_t* mask = p.kv_mask + (static_cast<long long>(head) * p.kv_blocks + kvb) * p.mask_words;
  int n = 0;
  for (int w = 0; w < p.mask_words; ++w) n += __popc(mask[w]);

  if (tid == 0) {
    mbar_init(&sm.kv_full, 1);
    mbar_init(&sm.qd_full[0], 1);
    mbar_init(&sm.qd_full[1], 1);
    mbar_init(&sm.sp_done, 1);
    mbar_init(&sm.dkv_done, 1);
    mbar_init(&sm.sp_free, kSoftmaxThreads);
    mbar_init(&sm.pd_ready, kSoftmaxThreads);
    sm.abort_flag = 0;
    fence_barrier_init();
  }
  if (tid < kBlock) {
    const long long s = static_cast<long long>(kvb) * kBlock + tid;
    sm.out_row[tid] = p.kv_slot_row != nullptr ? p.kv_slot_row[s] : s;
  }
  if (warp == 0) {
    tmem_alloc(&sm.tmem_base, kDkvTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  volatile int* abort_flag = &sm.abort_flag;
  MaskCursor cursor(mask, p.mask_words);
  const int kv_size = p.kv_sizes != nullptr ? p.kv_sizes[kvb] : kBlock;

  if (warp == 4) {
    // ------------------------------------------------------------ issuer: TMA loads and MMAs
    if (lane == 0 && n > 0) {
      auto load_stage = [&](int stage, int q_block) {
        mbar_expect_tx(&sm.qd_full[stage], 2 * kTileBytes);
        tma_load_tile(sm.q[stage], &p.q_map, &sm.qd_full[stage], head, q_block);
        tma_load_tile(sm.d_o[stage], &p.do_map, &sm.qd_full[stage], head, q_block);
      };
      mbar_expect_tx(&sm.kv_full, 2 * kTileBytes);
      tma_load_tile(sm.k, &p.k_map, &sm.kv_full, head, kvb);
      tma_load_tile(sm.v, &p.v_map, &sm.kv_full, head, kvb);
      for (int s = 0; s < 2 && s < n; ++s) load_stage(s, cursor.next());
      mbar_wait(&sm.kv_full, 0, abort_flag, p.status, 21);
      mbar_wait(&sm.qd_full[0], 0, abort_flag, p.status, 22);
      tc_fence_after();
      issue_nt_128(tmem, sm.q[0], sm.k);
      issue_nt_128(tmem + 64, sm.d_o[0], sm.v);
      umma_commit(&sm.sp_done);
      for (int j = 0; j < n; ++j) {
        const int b = j & 1;
        if (j + 1 < n) {
          mbar_wait(&sm.sp_free, j & 1, abort_flag, p.status, 28);
          mbar_wait(&sm.qd_full[b ^ 1], ((j + 1) >> 1) & 1, abort_flag, p.status, 26);
          tc_fence_after();
          issue_nt_128(tmem, sm.q[b ^ 1], sm.k);
          issue_nt_128(tmem + 64, sm.d_o[b ^ 1], sm.v);
          umma_commit(&sm.sp_done);
        }
        mbar_wait(&sm.pd_ready, j & 1, abort_flag, p.status, 29);
        tc_fence_after();
        issue_tt_128(tmem + 192, sm.d_o[b], sm.pt, j > 0);  // dV^T += dO^T P
        issue_tt_128(tmem + 128, sm.q[b], sm.dst, j > 0);   // dK^T += Q^T dS
        umma_commit(&sm.dkv_done);
        if (j + 2 < n) {
          // Stage b is free once this step (the newest commit on the barrier) has read Q_j, dO_j.
          mbar_wait(&sm.dkv_done, j & 1, abort_flag, p.status, 25);
          load_stage(b, cursor.next());
        }
      }
    }
  } else {
    // ------------------------------------------------------------ score math warps
    const float sl2 = p.scale * kLog2e;
    const long long head_stats = static_cast<long long>(head) * p.q_slots + row;
    // LSE and delta of this thread's query row, fetched one tile ahead.
    float lse_next = 0.f, delta_next = 0.f;
    if (n > 0) {
      const long long at = head_stats + static_cast<long long>(cursor.next()) * kBlock;
      lse_next = p.lse[at];
      delta_next = p.delta[at];
    }
    for (int j = 0; j < n; ++j) {
      const float lse2 = lse_next * kLog2e, delta = delta_next;
      if (j + 1 < n) {
        const long long at = head_stats + static_cast<long long>(cursor.next()) * kBlock;
        lse_next = p.lse[at];
        delta_next = p.delta[at];
      }
      mbar_wait(&sm.sp_done, j & 1, abort_flag, p.status, 23);
      tc_fence_after();
      uint32_t s_bits[32], dp_bits[32];
      VSA_TMEM_LD_16x32bx2_X32(s_bits, tmem + lane_base, 32);
      VSA_TMEM_LD_16x32bx2_X32(dp_bits, tmem + lane_base + 64, 32);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&sm.sp_free);
      const bool row_live = lse2 != -INFINITY;
      uint32_t p_packed[16], ds_packed[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float pr[2], ds[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const bool live = row_live && (half * 32 + i + e < kv_size);
          pr[e] = live ? fast_exp2(fmaf(__uint_as_float(s_bits[i + e]), sl2, -lse2)) : 0.f;
          ds[e] = pr[e] * (__uint_as_float(dp_bits[i + e]) - delta) * p.scale;
        }
        p_packed[i >> 1] = pack_bf16(pr[0], pr[1]);
        ds_packed[i >> 1] = pack_bf16(ds[0], ds[1]);
      }
      if (j > 0) {
        // Step j-1 has finished reading the P^T / dS^T buffers.
        mbar_wait(&sm.dkv_done, (j - 1) & 1, abort_flag, p.status, 25);
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t off = swizzled_offset(row, half * 4 + c);
        *reinterpret_cast<uint4*>(sm.pt + off) =
            make_uint4(p_packed[4 * c], p_packed[4 * c + 1], p_packed[4 * c + 2], p_packed[4 * c + 3]);
        *reinterpret_cast<uint4*>(sm.dst + off) =
            make_uint4(ds_packed[4 * c], ds_packed[4 * c + 1], ds_packed[4 * c + 2], ds_packed[4 * c + 3]);
      }
      fence_proxy_async_smem();
      mbar_arrive(&sm.pd_ready);
    }
    if (n > 0) {
      mbar_wait(&sm.dkv_done, (n - 1) & 1, abort_flag, p.status, 27);
      tc_fence_after();
    }
    const long long width = static_cast<long long>(p.heads) * kDim;
    const long long col = static_cast<long long>(head) * kDim + tid;
    float term = pool_term(p.dk_pool, p.pool_f32, p.kv_block_coarse, kvb, kv_size, width, col);
    store_grad_columns(n > 0, tmem + lane_base + 128, term, sm.out_row, p.kv_out_rows, p.dk, p.dk_f32,
                       p.f32_accumulate != 0, kvb, width, col);
    term = pool_term(p.dv_pool, p.pool_f32, p.kv_block_coarse, kvb, kv_size, width, col);
    store_grad_columns(n > 0, tmem + lane_base + 192, term, sm.out_row, p.kv_out_rows, p.dv, p.dv_f32,
                       p.f32_accumulate != 0, kvb, width, col);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kDkvTmemCols);
}

// Marks, for every (head, KV block), the query blocks whose list contains it.
__global__ void build_kv_mask_kernel(const int32_t* indices, const int32_t* counts, long long index_head_stride,
                                     long long count_head_stride, int capacity, int q_blocks, int kv_blocks,
                                     uint32_t* mask, int mask_words) {
  const int qb = blockIdx.x, head = blockIdx.y;
  const int n = counts[static_cast<long long>(head) * count_head_stride + qb];
  const int32_t* list = indices + static_cast<long long>(head) * index_head_stride +
                        static_cast<long long>(qb) * capacity;
  uint32_t* head_mask = mask + static_cast<long long>(head) * kv_blocks * mask_words;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const int kv = list[j];
    if (kv >= 0 && kv < kv_blocks)
      atomicOr(head_mask + static_cast<long long>(kv) * mask_words + (qb >> 5), 1u << (qb & 31));
  }
}

cudaError_t launch_build_kv_mask(const int32_t* indices, const int32_t* counts, long long index_head_stride,
                                 long long count_head_stride, int capacity, int heads, int q_blocks,
                                 int kv_blocks, uint32_t* mask, int mask_words, cudaStream_t stream) {
  const size_t bytes = static_cast<size_t>(heads) * kv_blocks * mask_words * sizeof(uint32_t);
  cudaError_t err = cudaMemsetAsync(mask, 0, bytes, stream);
  if (err != cudaSuccess) return err;
  dim3 grid(q_blocks, heads);
  build_kv_mask_kernel<<<grid, 128, 0, stream>>>(indices, counts, index_head_stride, count_head_stride, capacity,
                                                 q_blocks, kv_blocks, mask, mask_words);
  return cudaGetLastError();
}

cudaError_t launch_fine_bwd_dq(const FineBwdParams& params, cudaStream_t stream) {
  const size_t smem = sizeof(DqSmem) + 1024;
  cudaError_t err = cudaFuncSetAttribute(fine_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
  if (err != cudaSuccess) return err;
  dim3 grid(params.q_blocks, params.heads);
  fine_bwd_dq_kernel<<<grid, kThreads, smem, stream>>>(params);
  return cudaGetLastError();
}

cudaError_t launch_fine_bwd_dkv(const FineBwdParams& params, cudaStream_t stream) {
  const size_t smem = sizeof(DkvSmem);
  cudaError_t err = cudaFuncSetAttribute(fine_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
  if (err != cudaSuccess) return err;
  dim3 grid(params.kv_blocks, params.heads);
  fine_bwd_dkv_kernel<<<grid, kThreads, smem, stream>>>(params);
  return cudaGetLastError();
}

}  // namespace vsa
