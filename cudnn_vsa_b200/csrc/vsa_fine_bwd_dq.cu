// Block-sparse fine attention, backward, dQ kernel for sm_100a.
//
// One CTA owns one (query block, head) and walks the block's KV list two blocks ("a pair") at a
// time.  Every product puts 128 rows on the tensor core's M axis, the shape it runs at full rate:
//   S^T  = K Q^T        M = 128 keys of the pair,  N = 64 queries,  K = 128 head dims
//   dP^T = V dO^T       M = 128 keys,              N = 64 queries,  K = 128 head dims
//   dQ^T += K^T dS^T    M = 128 head dims,         N = 64 queries,  K = 128 keys
// With the keys on the TMEM lanes a thread of a score-math warpgroup owns one key and sees the
// 64 queries along its columns; the per-query LSE and delta are the same for every pair, so they
// sit in shared memory (pre-scaled) and are read as broadcasts.  P is recomputed from the saved
// LSE (natural log), dS^T = P^T * (dP^T - delta) * scale is written as BF16 rows [key][query],
// which is directly the MN-major B operand of the third product; K^T is the K pair read MN-major.
// Two warpgroups take alternate pairs, each with its own S^T / dP^T accumulators and dS^T buffer,
// one warp issues the score products and another the dQ products, synchronised only through
// mbarriers, so the exponentials of one pair run under the products of its neighbours and a wait
// of one kind of product never holds up the other.  K pair stages are
// held until their dQ product has read them (three stages), V pair stages only until dP^T (two).
// The epilogue adds the gradient that reaches a row through its block's pooled mean and scatters
// the rows to the caller's row order, skipping padding slots (reference vsa_core.py:23-30, 42-47;
// vsa_kernels.py:86-96, 161-176 adjoint).
#include "vsa_common.cuh"
#include "vsa_kernels.h"
#include "vsa_bwd_common.cuh"

namespace vsa {

namespace {

constexpr int kGroupThreads = 128;  // one score-math warpgroup
constexpr int kMathThreads = 256;   // warps 0..3: warpgroup 0 (even pairs), warps 4..7: warpgroup 1 (odd pairs)
constexpr int kThreads = 384;       // warp 8: issues the dQ products, warps 9 / 10: TMA loads of Q, dO, K / of V, warp 11: issues the score products
constexpr int kTmemCols = 512;      // per warpgroup g: S^T [128g, 128g+64)  dP^T [128g+64, 128g+128);  dQ^T [256,320)
constexpr uint32_t kColDq = 256;
constexpr int kKStages = 3;
constexpr int kVStages = 2;
constexpr int kPairBytes = 2 * kTileBytes;  // [dim half][tile of the pair][row][128 B]

struct DqSmem {  // placed at a 1024-byte aligned address; every tile offset is a multiple of 1024
  uint8_t q[kTileBytes];
  uint8_t d_o[kTileBytes];
  uint8_t k[kKStages][kPairBytes];
  uint8_t v[kVStages][kPairBytes];
  uint8_t ds[2][kTileBytes];  // per warpgroup: dS^T [128 keys][64 queries] BF16, 128-byte swizzle
  float neg_lse2[kBlock];     // -lse * log2(e) per query row (-inf for a row without keys)
  float delta[kBlock];
  long long out_row[kBlock];
  uint64_t qdo_full, k_full[kKStages], v_full[kVStages], k_free[kKStages], v_free[kVStages];
  uint64_t sp_done[2], sp_free[2], ds_ready[2], ds_free[2], dq_final;
  uint32_t tmem_base;
  int abort_flag;
};

// S^T or dP^T = A B^T: A = a K-major pair stage (128 rows), B = the first N rows of a K-major
// 64-row tile (N = the query block's valid rows rounded up to 16, carried by `idesc`); eight
// K=16 steps over the two 64-wide dim halves.
VSA_DEVICE void issue_scores(uint32_t tmem_d, uint32_t pair_lo, uint32_t tile_lo, uint32_t idesc) {
#pragma unroll
  for (int ks = 0; ks < 8; ++ks)
    umma_ss_lo(tmem_d, pair_lo + (ks >> 2) * (kTileBytes >> 4) + (ks & 3) * 2,
               tile_lo + (ks >> 2) * (kHalfTileBytes >> 4) + (ks & 3) * 2, idesc, ks > 0);
}

// dQ^T (+)= K^T dS^T over the keys of one or two blocks: A = the K pair read MN-major (16 keys =
// 2 KiB per step, dim halves 16 KiB apart), B = the first N queries of the dS^T rows [key][query]
// read MN-major.  `steps0` / `steps1`: K=16 steps that hold real keys of the first / second
// block (0 = block absent); dS^T is zero on padded keys, so their steps are not issued.  Full
// blocks take the straight-line path: the issuing thread pays for every instruction between MMAs.
VSA_DEVICE void issue_dq(uint32_t tmem_d, uint32_t k_mn_lo, uint32_t ds_lo, int steps0, int steps1, bool accumulate,
                         uint32_t idesc) {
  if (steps0 == 4 && (steps1 == 4 || steps1 == 0)) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) umma_ss_lo(tmem_d, k_mn_lo + ks * 128, ds_lo + ks * 128, idesc, accumulate || ks > 0);
    if (steps1) {
#pragma unroll
      for (int ks = 4; ks < 8; ++ks) umma_ss_lo(tmem_d, k_mn_lo + ks * 128, ds_lo + ks * 128, idesc, 1u);
    }
    return;
  }
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
    if (ks < steps0) umma_ss_lo(tmem_d, k_mn_lo + ks * 128, ds_lo + ks * 128, idesc, accumulate || ks > 0);
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
    if (ks < steps1) umma_ss_lo(tmem_d, k_mn_lo + (4 + ks) * 128, ds_lo + (4 + ks) * 128, idesc, 1u);
}

// dS^T of 32 queries of this thread's key from the S^T and dP^T accumulator bits.  kMasked: the
// chunk holds query columns at or beyond `q_n` that the products never wrote and that must come
// out as zero; a full chunk skips the per-element compare (the loop is bound by instruction
// issue).  A query row without keys has neg_lse2 = -inf: exp2(-inf) = 0.
template <bool kMasked>
VSA_DEVICE void ds_chunk(const uint32_t (&s_bits)[32], const uint32_t (&dp_bits)[32], bool live, int first_query,
                         int q_n, const float* neg_lse2, const float* delta, float sl2, float scale,
                         uint32_t* packed) {
#pragma unroll
  for (int e = 0; e < 32; e += 4) {
    const float4 nl = *reinterpret_cast<const float4*>(neg_lse2 + first_query + e);
    const float4 dl = *reinterpret_cast<const float4*>(delta + first_query + e);
    const float nls[4] = {nl.x, nl.y, nl.z, nl.w}, dls[4] = {dl.x, dl.y, dl.z, dl.w};
    float ds[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float pr = fast_exp2(fmaf(__uint_as_float(s_bits[e + u]), sl2, nls[u]));
      const float v = pr * (__uint_as_float(dp_bits[e + u]) - dls[u]) * scale;
      // A select: rows of an absent or padded key and unwritten columns may hold anything.
      ds[u] = (kMasked ? (live && first_query + e + u < q_n) : live) ? v : 0.f;
    }
    packed[e >> 1] = pack_bf16(ds[0], ds[1]);
    packed[(e >> 1) + 1] = pack_bf16(ds[2], ds[3]);
  }
}

}  // namespace

__global__ void __launch_bounds__(kThreads, 1) fine_bwd_dq_kernel(const __grid_constant__ FineBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  DqSmem& sm = *reinterpret_cast<DqSmem*>(smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qb = blockIdx.x, head = blockIdx.y;
  const int group = (warp >> 2) & 1;  // score-math warpgroup (warps 0..7 only)
  const int key = tid & 127;          // key of the pair owned by this thread (math role) / head dim (epilogue)
  const int n = p.counts[static_cast<long long>(head) * p.count_head_stride + qb];
  const int32_t* list = p.indices + static_cast<long long>(head) * p.index_head_stride +
                        static_cast<long long>(qb) * p.capacity;
  // Query rows the products cover: the block's valid rows rounded up to the MMA's N granularity.
  const int q_size = p.q_sizes != nullptr ? p.q_sizes[qb] : kBlock;
  const int q_n = q_size >= kBlock ? kBlock : (q_size <= 16 ? 16 : ((q_size + 15) & ~15));

  if (tid == 0) {
    mbar_init(&sm.qdo_full, 1);
    for (int i = 0; i < kKStages; ++i) {
      mbar_init(&sm.k_full[i], 1);
      mbar_init(&sm.k_free[i], 1);
    }
    for (int i = 0; i < kVStages; ++i) {
      mbar_init(&sm.v_full[i], 1);
      mbar_init(&sm.v_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.sp_done[i], 1);
      mbar_init(&sm.sp_free[i], kGroupThreads);
      mbar_init(&sm.ds_ready[i], kGroupThreads);
      mbar_init(&sm.ds_free[i], 1);
    }
    mbar_init(&sm.dq_final, 1);
    sm.abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&p.q_map);
    tma_prefetch_desc(&p.do_map);
    tma_prefetch_desc(&p.k_half_map);
    tma_prefetch_desc(&p.v_half_map);
  }
  if (tid < kBlock) {
    const long long s = static_cast<long long>(qb) * kBlock + tid;
    sm.out_row[tid] = p.q_slot_row != nullptr ? p.q_slot_row[s] : s;
    const float lse = p.lse[static_cast<long long>(head) * p.q_slots + s];
    sm.neg_lse2[tid] = lse == -INFINITY ? -INFINITY : -lse * kLog2eBwd;
    sm.delta[tid] = p.delta[static_cast<long long>(head) * p.q_slots + s];
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

  // Barrier discipline: a barrier is only ever waited on for its NEWEST commit or arrival round;
  // every barrier belongs to one buffer and the round after the awaited one cannot start before
  // the waiter has moved on.
  const int pairs = (n + 1) >> 1;
  if (warp == 9 || warp == 10) {
    // ------------------------------------------------------------ producers: TMA loads
    // K and V have a producer warp each: V stages are released after dP^T, K stages only after
    // the dQ product, and one in-order loop would hold each load behind the other's wait.
    if (lane == 0 && n > 0) {
      const bool is_k = warp == 9;
      if (is_k) {
        mbar_expect_tx(&sm.qdo_full, 2 * kTileBytes);
        tma_load_tile(sm.q, &p.q_map, &sm.qdo_full, head, qb);
        tma_load_tile(sm.d_o, &p.do_map, &sm.qdo_full, head, qb);
      }
      const CUtensorMap* map = is_k ? &p.k_half_map : &p.v_half_map;
      const int stages = is_k ? kKStages : kVStages;
      int stage = 0;
      uint32_t round = 0;  // parity of the release awaited before refilling the stage
      for (int i = 0; i < pairs; ++i) {
        const int count = (2 * i + 1 < n) ? 2 : 1;
        uint64_t* full = is_k ? &sm.k_full[stage] : &sm.v_full[stage];
        uint8_t* dst = is_k ? sm.k[stage] : sm.v[stage];
        if (i >= stages) mbar_wait(is_k ? &sm.k_free[stage] : &sm.v_free[stage], round, abort_flag, p.status, 12);
        mbar_expect_tx(full, count * kTileBytes);
        for (int t = 0; t < count; ++t)
          for (int h = 0; h < 2; ++h) tma_load_half(dst + h * kTileBytes + t * kHalfTileBytes, map, full, head, list[2 * i + t], h);
        if (++stage == stages) {
          stage = 0;
          if (i >= stages) round ^= 1;
        }
      }
    }
  } else if (warp == 11) {
    // ------------------------------------------------------------ issuer of the score products
    // Two issuing warps, one per kind of product, synchronised only through the barriers: the
    // score products of pair j + 2 start as soon as their operands have landed and warpgroup
    // j & 1 has pulled pair j out of the accumulators, whatever the dQ products are waiting for.
    // The whole warp walks the loop (uniform control flow and addresses); one elected lane
    // issues the MMAs and commits.
    if (n > 0) {
      const bool leader = elect_one();
      const uint32_t q_lo = umma_desc_lo(smem_u32(sm.q), 16);
      const uint32_t do_lo = umma_desc_lo(smem_u32(sm.d_o), 16);
      const uint32_t k_lo0 = umma_desc_lo(smem_u32(sm.k[0]), 16);
      const uint32_t v_lo0 = umma_desc_lo(smem_u32(sm.v[0]), 16);
      constexpr uint32_t kPairLo = kPairBytes >> 4;
      int s_k = 0, s_v = 0;                   // stages of the next score products
      uint32_t s_k_phase = 0, s_v_phase = 0;  // parities of those stages' current fills
      const uint32_t idesc = umma_idesc(128, q_n, 0, 0);
      mbar_wait(&sm.qdo_full, 0, abort_flag, p.status, 11);
      for (int j = 0; j < pairs; ++j) {
        if (j >= 2) mbar_wait(&sm.sp_free[j & 1], ((j >> 1) - 1) & 1, abort_flag, p.status, 17);
        mbar_wait(&sm.k_full[s_k], s_k_phase, abort_flag, p.status, 15);
        tc_fence_after();
        if (leader) issue_scores(tmem + (j & 1) * 128, k_lo0 + s_k * kPairLo, q_lo, idesc);
        mbar_wait(&sm.v_full[s_v], s_v_phase, abort_flag, p.status, 19);
        tc_fence_after();
        if (leader) {
          issue_scores(tmem + (j & 1) * 128 + 64, v_lo0 + s_v * kPairLo, do_lo, idesc);
          umma_commit(&sm.sp_done[j & 1]);
          umma_commit(&sm.v_free[s_v]);
        }
        if (++s_k == kKStages) {
          s_k = 0;
          s_k_phase ^= 1;
        }
        if (++s_v == kVStages) {
          s_v = 0;
          s_v_phase ^= 1;
        }
      }
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------ issuer of the dQ products
    if (n > 0) {
      const bool leader = elect_one();
      const uint32_t k_mn_lo0 = umma_desc_lo(smem_u32(sm.k[0]), kTileBytes);
      const uint32_t ds_lo0 = umma_desc_lo(smem_u32(sm.ds[0]), kHalfTileBytes);
      constexpr uint32_t kPairLo = kPairBytes >> 4, kDsLo = kTileBytes >> 4;
      int d_k = 0;  // K stage of the next dQ product
      const uint32_t idesc = umma_idesc(128, q_n, 1, 1);
      // K=16 steps that hold real keys, per block of the pair; looked up one pair ahead so the
      // two dependent loads never sit between a completed wait and its products.
      auto steps_of = [&](int i, int& s0, int& s1) {
        s0 = 4;
        s1 = (2 * i + 1 < n) ? 4 : 0;
        if (p.kv_sizes != nullptr) {
          s0 = (p.kv_sizes[list[2 * i]] + 15) >> 4;
          s0 = s0 < 1 ? 1 : s0;
          if (s1) s1 = (p.kv_sizes[list[2 * i + 1]] + 15) >> 4;
        }
      };
      int steps0 = 4, steps1 = 0;
      steps_of(0, steps0, steps1);
      for (int i = 0; i < pairs; ++i) {
        const int now0 = steps0, now1 = steps1;
        if (i + 1 < pairs) steps_of(i + 1, steps0, steps1);
        mbar_wait(&sm.ds_ready[i & 1], (i >> 1) & 1, abort_flag, p.status, 18);
        tc_fence_after();
        if (leader) {
          issue_dq(tmem + kColDq, k_mn_lo0 + d_k * kPairLo, ds_lo0 + (i & 1) * kDsLo, now0, now1, i > 0, idesc);
          umma_commit(&sm.k_free[d_k]);
          umma_commit(&sm.ds_free[i & 1]);
        }
        if (++d_k == kKStages) d_k = 0;
      }
      if (leader) umma_commit(&sm.dq_final);
    }
  } else {
    // ------------------------------------------------------------ score math warpgroups
    const uint32_t tmem_s = tmem + lane_base + group * 128;
    uint8_t* ds_row = sm.ds[group] + key * 128;
    const int tile = key >> 6, key_in_block = key & 63;
    const float scale = p.scale, sl2 = p.scale * kLog2eBwd;
    // The valid length of a block comes from two dependent global loads (list, then sizes).  They
    // are software-pipelined over two rounds - the block id is fetched two rounds ahead, the size
    // one round ahead from an id that is already in a register - so no load is issued behind the
    // one it depends on.
    int size_next = kBlock;
    if (p.kv_sizes != nullptr && 2 * group + tile < n) size_next = p.kv_sizes[list[2 * group + tile]];
    int block_next = (p.kv_sizes != nullptr && 2 * group + 4 + tile < n) ? list[2 * group + 4 + tile] : 0;
    for (int i = group; i < pairs; i += 2) {
      const bool live = (2 * i + tile < n) && key_in_block < size_next;
      if (p.kv_sizes != nullptr) {
        if (2 * i + 4 + tile < n) size_next = p.kv_sizes[block_next];
        if (2 * i + 8 + tile < n) block_next = list[2 * i + 8 + tile];
      }
      mbar_wait(&sm.sp_done[group], (i >> 1) & 1, abort_flag, p.status, 13);
      tc_fence_after();
      uint32_t packed[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        if (c * 32 >= q_n) break;  // a short query block has no second half
        uint32_t s_bits[32], dp_bits[32];
        VSA_TMEM_LD_32x32b_X32(s_bits, tmem_s + c * 32);
        VSA_TMEM_LD_32x32b_X32(dp_bits, tmem_s + 64 + c * 32);
        tmem_wait_ld();
        if ((c + 1) * 32 >= q_n) {
          // All of S^T and dP^T is in registers: the accumulators may be overwritten.
          tc_fence_before();
          mbar_arrive(&sm.sp_free[group]);
        }
        if ((c + 1) * 32 <= q_n)
          ds_chunk<false>(s_bits, dp_bits, live, c * 32, q_n, sm.neg_lse2, sm.delta, sl2, scale, packed + c * 16);
        else
          ds_chunk<true>(s_bits, dp_bits, live, c * 32, q_n, sm.neg_lse2, sm.delta, sl2, scale, packed + c * 16);
      }
      // The dQ product of this warpgroup's previous pair has finished reading the dS^T buffer.
      if (i >= 2) mbar_wait(&sm.ds_free[group], ((i >> 1) - 1) & 1, abort_flag, p.status, 14);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c * 8 >= q_n) break;  // the product reads q_n queries of every row
        *reinterpret_cast<uint4*>(ds_row + ((c ^ (key & 7)) << 4)) =
            make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&sm.ds_ready[group]);
    }
  }

  // ---------------------------------------------------------------- epilogue
  if (warp < 8) {
    if (n > 0) {
      mbar_wait(&sm.dq_final, 0, abort_flag, p.status, 16);
      tc_fence_after();
    }
    // Thread = head dim `key`; warpgroup g takes query rows [32g, 32g+32), of which only the
    // block's valid rows are written.  A warp store covers 32 consecutive elements of one row.
    const long long width = static_cast<long long>(p.heads) * kDim;
    const long long col = static_cast<long long>(head) * kDim + key;
    if (group * 32 < q_size) {
      const float term = pool_term(p.dq_pool, p.pool_f32, p.q_block_coarse, qb, q_size, width, col);
      uint32_t bits[32] = {};
      if (n > 0) {
        VSA_TMEM_LD_32x32b_X32(bits, tmem + lane_base + kColDq + group * 32);
        tmem_wait_ld();
      }
      if (p.dq_f32 != nullptr) {
        // Running FP32 dQ of the ring: every old value of the chunk is fetched before the first
        // store, so the loads are in flight together.
        float* base = p.dq_f32 + (static_cast<long long>(qb) * kBlock + group * 32) * width + col;
        float old[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) old[i] = (p.f32_accumulate && group * 32 + i < q_size) ? base[i * width] : 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (group * 32 + i < q_size) base[i * width] = old[i] + (__uint_as_float(bits[i]) + term);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int r = group * 32 + i;
          const long long row = sm.out_row[r];
          if (r < q_size && row >= 0 && row < p.q_out_rows)
            p.dq[row * p.out_row_stride + head * p.out_head_stride + key] = __float2bfloat16(__uint_as_float(bits[i]) + term);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
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

}  // namespace vsa
