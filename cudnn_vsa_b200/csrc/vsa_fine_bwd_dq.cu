// Block-sparse fine attention, backward, dQ kernel for sm_100a.
//
// A tile is one (query block, head): the CTA walks the block's KV list two blocks ("a pair") at a
// time.  The kernel is persistent - one CTA per SM takes tiles in head-major order from a work
// counter; the thread that loads Q, dO and K publishes each tile's head, block, list length and
// valid rows in a small shared-memory queue that the other roles read in order - so barriers,
// tensor memory and the stage rings are set up once, the loads of the next tile run under the
// last pairs and the epilogue of the current one, and the per-row data of the next tile (LSE,
// delta, output rows) is fetched while the epilogue stores.  Every product puts 128 rows on the tensor core's M axis, the shape it runs at full rate:
//   S^T  = K Q^T        M = 128 keys of the pair,  N = 64 queries,  K = 128 head dims
//   dP^T = V dO^T       M = 128 keys,              N = 64 queries,  K = 128 head dims
//   dQ^T += K^T dS^T    M = 128 head dims,         N = 64 queries,  K = 128 keys
// With the keys on the TMEM lanes a thread of a score-math warpgroup owns one key and sees the
// 64 queries along its columns; the per-query LSE and delta are the same for every pair, so they
// sit in shared memory (pre-scaled) and are read as broadcasts.  P is recomputed from the saved
// LSE (natural log), dS^T = P^T * (dP^T - delta) * scale is written as BF16 rows [key][query],
// which is directly the MN-major B operand of the third product; K^T is the K pair read MN-major.
// Both score-math warpgroups work on every pair - a thread owns one key and 32 of the 64 queries -
// because the latency of that step is on the critical path: a K stage is only refilled after the
// pair's dQ product, which waits for the pair's dS^T, and there is room for three K stages.  Two
// sets of S^T / dP^T accumulators and two dS^T buffers alternate between pairs; one warp issues
// the score products and another the dQ products, synchronised only through mbarriers, so the
// exponentials of one pair run under the products of its neighbours and a wait of one kind of
// product never holds up the other.  K pair stages are
// held until their dQ product has read them (three stages), V pair stages only until dP^T (two).
// The epilogue adds the gradient that reaches a row through its block's pooled mean and scatters
// the rows to the caller's row order, skipping padding slots (reference vsa_core.py:23-30, 42-47;
// vsa_kernels.py:86-96, 161-176 adjoint).
#include "vsa_common.cuh"
#include "vsa_kernels.h"
#include "vsa_bwd_common.cuh"

namespace vsa {

namespace {

constexpr int kMathThreads = 256;   // warps 0..3 / 4..7: queries 0..31 / 32..63 of every pair's S^T and dP^T
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
  long long out_row[2][kBlock];  // by tile parity: the next tile's rows are staged while this tile's are stored
  uint64_t qdo_full, qdo_free, k_full[kKStages], v_full[kVStages], k_free[kKStages], v_free[kVStages];
  uint64_t sp_done[2], sp_free[2], ds_ready[2], ds_free[2], dq_final, dq_free;
  TileQueue tiles;
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
  const int group = (warp >> 2) & 1;  // score-math warpgroup (warps 0..7 only)
  const int key = tid & 127;          // key of the pair owned by this thread (math role) / head dim (epilogue)
  const int tiles = p.q_blocks * p.heads;  // tile t = (head, query block), head-major
  // Consumers of the tile queue: the V producer, the two issuing warps, the eight math warps.
  constexpr int kQueueConsumers = 11;
  // Query rows the products cover: the block's valid rows rounded up to the MMA's N granularity.
  auto covered_rows = [](int q_size) -> int {
    return q_size >= kBlock ? kBlock : (q_size <= 16 ? 16 : ((q_size + 15) & ~15));
  };
  auto list_of = [&](const TileInfo& t) -> const int32_t* {
    return p.indices + static_cast<long long>(t.head) * p.index_head_stride + static_cast<long long>(t.block) * p.capacity +
           t.aux3;
  };

  if (tid == 0) {
    mbar_init(&sm.qdo_full, 1);
    mbar_init(&sm.qdo_free, 1);
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
      mbar_init(&sm.sp_free[i], kMathThreads);
      mbar_init(&sm.ds_ready[i], kMathThreads);
      mbar_init(&sm.ds_free[i], 1);
    }
    mbar_init(&sm.dq_final, 1);
    mbar_init(&sm.dq_free, kMathThreads);
    tile_queue_init(sm.tiles, kQueueConsumers);
    sm.abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&p.q_map);
    tma_prefetch_desc(&p.do_map);
    tma_prefetch_desc(&p.k_half_map);
    tma_prefetch_desc(&p.v_half_map);
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
  static_assert(kKStages == 3 && kVStages == 2, "the stage rings below are written for 3 K and 2 V stages");

  // Barrier discipline: a barrier is only ever waited on for its NEWEST commit or arrival round;
  // every barrier belongs to one buffer and the round after the awaited one cannot start before
  // the waiter has moved on.  Pairs are numbered through all tiles of the CTA (`g` below): pair
  // g uses accumulator set, dS^T buffer and math warpgroup g & 1, V stage g & 1 and K stage
  // g % 3, whatever tile it belongs to; `used` counts the non-empty tiles so far.  Every role
  // skips empty tiles.
  if (warp == 9) {
    // ------------------------------------------------------------ producer of Q, dO and K; scheduler
    // K and V have a producer warp each: V stages are released after dP^T, K stages only after
    // the dQ product, and one in-order loop would hold each load behind the other's wait.
    if (lane == 0) {
      Ring3 ring;
      int used = 0;
      // Tile numbers: the block index first, then the work counter.  The next number is taken
      // only when the last loads of the current tile are about to be issued - a CTA that held
      // tiles in reserve would keep them from idle SMs at the end of the launch, and one list
      // can be a hundred times longer than another - which still leaves the counter and the
      // tile's list length a few pairs of time to arrive.
      auto info_of = [&](int t) -> TileInfo {
        if (t >= tiles) return TileInfo{0, 0, -1};
        const int head = t / p.q_blocks, qb = t - head * p.q_blocks;
        // aux = valid rows of the query block, aux2 = row of its pooled-mean gradient (-1 = none),
        // aux3 = first entry of the list's sub-range.
        int pool_row = -1;
        if (p.dq_pool != nullptr) pool_row = p.pool_f32 ? qb : (p.q_block_coarse != nullptr ? p.q_block_coarse[qb] : -1);
        const int q_size = p.q_sizes != nullptr ? p.q_sizes[qb] : kBlock;
        const long long row = static_cast<long long>(head) * p.count_head_stride + qb;
        if (p.list_bounds == nullptr) return TileInfo{head, qb, p.counts[row], q_size, pool_row, 0};
        const int32_t* bounds = p.list_bounds + row * p.bounds_stride;
        const int begin = bounds[0];
        return TileInfo{head, qb, bounds[1] - begin, q_size, pool_row, begin};
      };
      auto take_number = [&]() -> int { return static_cast<int>(gridDim.x + atomicAdd(p.tile_counter, 1u)); };
      TileInfo cur = info_of(static_cast<int>(blockIdx.x));
      for (int seq = 0;; ++seq) {
        tile_publish(sm.tiles, seq, cur, abort_flag, p.status, 40);
        if (cur.count < 0 || *abort_flag) break;  // end of the tiles, or a wait gave up: start no further loads
        const TileInfo now = cur;
        const int n = now.count;
        if (n == 0) {
          cur = info_of(take_number());
          continue;
        }
        const int32_t* list = list_of(now);
        const int pairs = (n + 1) >> 1;
        // Q and dO have one buffer: it is free once the previous tile's last score products are done.
        if (used >= 1) mbar_wait(&sm.qdo_free, (used - 1) & 1, abort_flag, p.status, 38);
        mbar_expect_tx(&sm.qdo_full, 2 * kTileBytes);
        tma_load_tile(sm.q, &p.q_map, &sm.qdo_full, now.head, now.block);
        tma_load_tile(sm.d_o, &p.do_map, &sm.qdo_full, now.head, now.block);
        const int claim_at = pairs > kKStages ? pairs - kKStages : 0;
        int t_next = tiles;
        for (int i = 0; i < pairs; ++i) {
          if (i == claim_at) t_next = take_number();
          const int count = (2 * i + 1 < n) ? 2 : 1;
          const int stage = ring.stage;
          if (ring.round >= 1) mbar_wait(&sm.k_free[stage], ring.phase ^ 1, abort_flag, p.status, 12);
          mbar_expect_tx(&sm.k_full[stage], count * kTileBytes);
          for (int t = 0; t < count; ++t)
            for (int h = 0; h < 2; ++h)
              tma_load_half(sm.k[stage] + h * kTileBytes + t * kHalfTileBytes, &p.k_half_map, &sm.k_full[stage], now.head,
                            list[2 * i + t], h);
          ring.advance();
        }
        ++used;
        cur = info_of(t_next);
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------ producer of V
    if (lane == 0) {
      int g = 0;
      TileInfo info;
      for (int seq = 0; tile_take(sm.tiles, seq, info, abort_flag, p.status, 41); ++seq) {
        tile_release(sm.tiles, seq);
        const int n = info.count;
        if (n == 0) continue;
        const int32_t* list = list_of(info);
        const int pairs = (n + 1) >> 1;
        for (int i = 0; i < pairs; ++i, ++g) {
          const int count = (2 * i + 1 < n) ? 2 : 1;
          const int stage = g & 1;
          if (g >= 2) mbar_wait(&sm.v_free[stage], ((g >> 1) - 1) & 1, abort_flag, p.status, 20);
          mbar_expect_tx(&sm.v_full[stage], count * kTileBytes);
          for (int t = 0; t < count; ++t)
            for (int h = 0; h < 2; ++h)
              tma_load_half(sm.v[stage] + h * kTileBytes + t * kHalfTileBytes, &p.v_half_map, &sm.v_full[stage], info.head,
                            list[2 * i + t], h);
        }
      }
    }
  } else if (warp == 11) {
    // ------------------------------------------------------------ issuer of the score products
    // Two issuing warps, one per kind of product, synchronised only through the barriers: the
    // score products of pair g + 2 start as soon as their operands have landed and warpgroup
    // g & 1 has pulled pair g out of the accumulators, whatever the dQ products are waiting for.
    // The whole warp walks the loop (uniform control flow and addresses); one elected lane
    // issues the MMAs and commits.
    const bool leader = elect_one();
    const uint32_t q_lo = umma_desc_lo(smem_u32(sm.q), 16);
    const uint32_t do_lo = umma_desc_lo(smem_u32(sm.d_o), 16);
    const uint32_t k_lo0 = umma_desc_lo(smem_u32(sm.k[0]), 16);
    const uint32_t v_lo0 = umma_desc_lo(smem_u32(sm.v[0]), 16);
    constexpr uint32_t kPairLo = kPairBytes >> 4;
    Ring3 ring;  // K stage of the next score products
    int g = 0, used = 0;
    TileInfo info;
    for (int seq = 0; __all_sync(0xffffffffu, tile_take(sm.tiles, seq, info, abort_flag, p.status, 42)); ++seq) {
      if (leader) tile_release(sm.tiles, seq);  // after the vote, so every lane has read the entry
      const int n = info.count;
      if (n == 0) continue;
      const int pairs = (n + 1) >> 1;
      const uint32_t idesc = umma_idesc(128, covered_rows(info.aux), 0, 0);
      mbar_wait(&sm.qdo_full, used & 1, abort_flag, p.status, 11);
      for (int j = 0; j < pairs; ++j, ++g) {
        const int set = g & 1;
        if (g >= 2) mbar_wait(&sm.sp_free[set], ((g >> 1) - 1) & 1, abort_flag, p.status, 17);
        mbar_wait(&sm.k_full[ring.stage], ring.phase, abort_flag, p.status, 15);
        tc_fence_after();
        if (leader) issue_scores(tmem + set * 128, k_lo0 + ring.stage * kPairLo, q_lo, idesc);
        mbar_wait(&sm.v_full[set], (g >> 1) & 1, abort_flag, p.status, 19);
        tc_fence_after();
        if (leader) {
          issue_scores(tmem + set * 128 + 64, v_lo0 + set * kPairLo, do_lo, idesc);
          umma_commit(&sm.sp_done[set]);
          umma_commit(&sm.v_free[set]);
          if (j + 1 == pairs) umma_commit(&sm.qdo_free);  // Q and dO have been read for the last time
        }
        ring.advance();
      }
      ++used;
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------ issuer of the dQ products
    const bool leader = elect_one();
    const uint32_t k_mn_lo0 = umma_desc_lo(smem_u32(sm.k[0]), kTileBytes);
    const uint32_t ds_lo0 = umma_desc_lo(smem_u32(sm.ds[0]), kHalfTileBytes);
    constexpr uint32_t kPairLo = kPairBytes >> 4, kDsLo = kTileBytes >> 4;
    int d_k = 0;  // K stage of the next dQ product
    int g = 0, used = 0;
    TileInfo info;
    for (int seq = 0; __all_sync(0xffffffffu, tile_take(sm.tiles, seq, info, abort_flag, p.status, 43)); ++seq) {
      if (leader) tile_release(sm.tiles, seq);
      const int n = info.count;
      if (n == 0) continue;
      const int pairs = (n + 1) >> 1;
      const int32_t* list = list_of(info);
      const uint32_t idesc = umma_idesc(128, covered_rows(info.aux), 1, 1);
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
      // The first product of a tile overwrites dQ^T: the epilogue of the previous tile must have read it.
      if (used >= 1) mbar_wait(&sm.dq_free, (used - 1) & 1, abort_flag, p.status, 39);
      for (int i = 0; i < pairs; ++i, ++g) {
        const int now0 = steps0, now1 = steps1;
        if (i + 1 < pairs) steps_of(i + 1, steps0, steps1);
        const int set = g & 1;
        mbar_wait(&sm.ds_ready[set], (g >> 1) & 1, abort_flag, p.status, 18);
        tc_fence_after();
        if (leader) {
          issue_dq(tmem + kColDq, k_mn_lo0 + d_k * kPairLo, ds_lo0 + set * kDsLo, now0, now1, i > 0, idesc);
          umma_commit(&sm.k_free[d_k]);
          umma_commit(&sm.ds_free[set]);
          if (i + 1 == pairs) umma_commit(&sm.dq_final);
        }
        if (++d_k == kKStages) d_k = 0;
      }
      ++used;
    }
  } else {
    // ------------------------------------------------------------ score math warpgroups and epilogue
    // Thread = key `key` of the pair (TMEM lane); warpgroup `group` takes queries [32 group, 32 group + 32).
    uint8_t* ds_row0 = sm.ds[0] + key * 128;
    const int tile = key >> 6, key_in_block = key & 63;
    const float scale = p.scale, sl2 = p.scale * kLog2eBwd;
    const long long width = static_cast<long long>(p.heads) * kDim;

    // What a tile needs before its first pair is fetched while the previous tile's epilogue runs:
    // LSE, delta and output row of query row `tid` (threads 0..63) into registers, staged into
    // shared memory before the epilogue's first barrier, and the first steps of the block-size
    // lookups below.  The valid length of a block comes from two dependent global loads (list,
    // then sizes); they are software-pipelined over two pairs - the block id is fetched two
    // pairs ahead, the size one pair ahead from an id that is already in a register - so no
    // load is issued behind the one it depends on.  Between tiles the ids are fetched before
    // the epilogue and the first size after it.
    float pre_lse = 0.f, pre_delta = 0.f;
    long long pre_row = 0;
    int size_next = kBlock, block_next = 0, block_first = -1;
    auto fetch_rows_and_ids = [&](const TileInfo& t) {
      if (tid < kBlock) {
        const long long s = static_cast<long long>(t.block) * kBlock + tid;
        pre_row = p.q_slot_row != nullptr ? p.q_slot_row[s] : s;
        pre_lse = p.lse[static_cast<long long>(t.head) * p.q_slots + s];
        pre_delta = p.delta[static_cast<long long>(t.head) * p.q_slots + s];
      }
      const int32_t* list = list_of(t);
      block_first = -1;
      block_next = 0;
      if (p.kv_sizes != nullptr) {
        if (tile < t.count) block_first = list[tile];
        if (2 + tile < t.count) block_next = list[2 + tile];
      }
    };
    auto stage_rows = [&](int parity) {
      if (tid < kBlock) {
        sm.out_row[parity][tid] = pre_row;
        sm.neg_lse2[tid] = pre_lse == -INFINITY ? -INFINITY : -pre_lse * kLog2eBwd;
        sm.delta[tid] = pre_delta;
      }
    };
    auto fetch_first_size = [&]() { size_next = block_first >= 0 ? p.kv_sizes[block_first] : kBlock; };

    int g0 = 0;    // pairs of the tiles before the current one
    int used = 0;  // non-empty tiles before the current one
    TileInfo cur;
    // The 256 threads go on only together: they meet at named barriers between tiles.
    bool have = named_barrier_all(1, kMathThreads, tile_take(sm.tiles, 0, cur, abort_flag, p.status, 44));
    if (lane == 0) tile_release(sm.tiles, 0);
    if (have) {
      fetch_rows_and_ids(cur);
      stage_rows(0);
      fetch_first_size();
      named_barrier(1, kMathThreads);
    }
    for (int seq = 0; have; ++seq) {
      const int n = cur.count, head = cur.head, qb = cur.block, q_size = cur.aux;
      const int q_n = covered_rows(q_size);
      const int pairs = (n + 1) >> 1;
      const int32_t* list = list_of(cur);
      // This warpgroup's queries: none when the block is that short, else all 32 or a masked chunk.
      const bool has_queries = group * 32 < q_n, full_chunk = (group + 1) * 32 <= q_n;
      for (int i = 0; i < pairs; ++i) {
        const int g = g0 + i, set = g & 1;
        const bool live = (2 * i + tile < n) && key_in_block < size_next;
        if (p.kv_sizes != nullptr) {
          if (2 * i + 2 + tile < n) size_next = p.kv_sizes[block_next];
          if (2 * i + 4 + tile < n) block_next = list[2 * i + 4 + tile];
        }
        mbar_wait(&sm.sp_done[set], (g >> 1) & 1, abort_flag, p.status, 13);
        tc_fence_after();
        uint32_t packed[16];
        if (has_queries) {
          uint32_t s_bits[32], dp_bits[32];
          const uint32_t tmem_s = tmem + lane_base + set * 128 + group * 32;
          VSA_TMEM_LD_32x32b_X32(s_bits, tmem_s);
          VSA_TMEM_LD_32x32b_X32(dp_bits, tmem_s + 64);
          tmem_wait_ld();
          // This thread's part of S^T and dP^T is in registers: the accumulators may be overwritten
          // once all 256 threads have said so.
          tc_fence_before();
          mbar_arrive(&sm.sp_free[set]);
          if (full_chunk)
            ds_chunk<false>(s_bits, dp_bits, live, group * 32, q_n, sm.neg_lse2, sm.delta, sl2, scale, packed);
          else
            ds_chunk<true>(s_bits, dp_bits, live, group * 32, q_n, sm.neg_lse2, sm.delta, sl2, scale, packed);
        } else {
          mbar_arrive(&sm.sp_free[set]);
        }
        // The dQ product of the pair before last has finished reading this dS^T buffer.
        if (g >= 2) mbar_wait(&sm.ds_free[set], ((g >> 1) - 1) & 1, abort_flag, p.status, 14);
        if (has_queries) {
          uint8_t* ds_row = ds_row0 + set * kTileBytes;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if ((group * 4 + c) * 8 >= q_n) break;  // the product reads q_n queries of every row
            *reinterpret_cast<uint4*>(ds_row + (((group * 4 + c) ^ (key & 7)) << 4)) =
                make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
          }
          fence_proxy_async_smem();
        }
        tc_fence_before();
        mbar_arrive(&sm.ds_ready[set]);
      }

      // The next tile, and the loads it starts with, under this tile's epilogue.
      TileInfo next;
      const bool have_next =
          named_barrier_all(1, kMathThreads, tile_take(sm.tiles, seq + 1, next, abort_flag, p.status, 45));
      if (lane == 0) tile_release(sm.tiles, seq + 1);
      if (have_next) fetch_rows_and_ids(next);

      // -------------------------------------------------------------- epilogue of the tile
      // Thread = head dim `key`; warpgroup g holds query rows [32g, 32g+32) of dQ^T.  The tile is
      // turned through shared memory (the dS^T buffers are idle: every dQ product of the tile has
      // completed) so that global memory sees 16-byte stores of whole row segments; only the
      // block's valid rows are written.
      const long long col = static_cast<long long>(head) * kDim + key;
      // (An empty tile adds nothing to a running FP32 sum.)
      const bool add_nothing = n == 0 && p.dq_f32 != nullptr && p.f32_accumulate != 0 && cur.aux2 < 0;
      const bool rows_here = group * 32 < q_size && !add_nothing;
      // Gradient that reaches the rows through the block's pooled mean, already divided by its size.
      float term = 0.f;
      if (cur.aux2 >= 0) {
        const long long at = static_cast<long long>(cur.aux2) * width + col;
        term = p.pool_f32 ? static_cast<const float*>(p.dq_pool)[at]
                          : __bfloat162float(static_cast<const __nv_bfloat16*>(p.dq_pool)[at]);
        term *= 1.f / static_cast<float>(q_size > 1 ? q_size : 1);
      }
      uint32_t bits[32] = {};
      if (n > 0) {
        mbar_wait(&sm.dq_final, used & 1, abort_flag, p.status, 16);
        tc_fence_after();
        if (rows_here) {
          VSA_TMEM_LD_32x32b_X32(bits, tmem + lane_base + kColDq + group * 32);
          tmem_wait_ld();
        }
        // dQ^T is in registers (or not needed): the next tile's first dQ product may overwrite it.
        tc_fence_before();
        mbar_arrive(&sm.dq_free);
      }
      const bool f32_out = p.dq_f32 != nullptr;
      if (rows_here) {
        if (f32_out) {
          float* turn = reinterpret_cast<float*>(sm.ds[0]) + group * 32 * kDim + key;  // [64 rows][128 dims] FP32
#pragma unroll
          for (int i = 0; i < 32; ++i) turn[i * kDim] = __uint_as_float(bits[i]) + term;
        } else {
          __nv_bfloat16* turn = reinterpret_cast<__nv_bfloat16*>(sm.ds[0]) + group * 32 * kDim + key;  // [64][128] BF16
#pragma unroll
          for (int i = 0; i < 32; ++i) turn[i * kDim] = __float2bfloat16(__uint_as_float(bits[i]) + term);
        }
      }
      if (have_next) stage_rows((seq + 1) & 1);  // nobody reads neg_lse2 / delta any more
      named_barrier(1, kMathThreads);
      const int math_tid = tid;  // 0..255
      if (add_nothing) {
      } else if (f32_out) {
        // Running FP32 dQ of the ring: rows of 512 bytes, a float4 per thread and step.  Adding to
        // the running sum is a vector reduction performed by the memory system: nothing is read
        // back, so no load latency sits in the epilogue.  Every element has one writer per launch
        // and launches are ordered by the stream, so the sum is the same as read-add-write.
        const float4* turn = reinterpret_cast<const float4*>(sm.ds[0]);
        float4* base = reinterpret_cast<float4*>(p.dq_f32 + static_cast<long long>(qb) * kBlock * width +
                                                 static_cast<long long>(head) * kDim);
        const long long row_vecs = width / 4;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int v = math_tid + j * kMathThreads, r = v >> 5, c = v & 31;
          if (r >= q_size) break;
          if (p.f32_accumulate)
            atomicAdd(base + r * row_vecs + c, turn[v]);
          else
            base[r * row_vecs + c] = turn[v];
        }
      } else {
        const uint4* turn = reinterpret_cast<const uint4*>(sm.ds[0]);
        const long long* out_row = sm.out_row[seq & 1];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int v = math_tid + j * kMathThreads, r = v >> 4, c = v & 15;
          const long long row = out_row[r];
          if (r < q_size && row >= 0 && row < p.q_out_rows)
            *reinterpret_cast<uint4*>(p.dq + row * p.out_row_stride + head * p.out_head_stride + c * 8) = turn[v];
        }
      }
      if (have_next) fetch_first_size();
      // The turning buffer is the next tile's dS^T buffer again.
      named_barrier(1, kMathThreads);
      g0 += pairs;
      if (n > 0) ++used;
      cur = next;
      have = have_next;
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
  // One CTA per SM (a CTA takes a whole SM's shared and tensor memory); fewer when there are fewer tiles.
  int device = 0, sms = 0;
  if ((err = cudaGetDevice(&device)) != cudaSuccess) return err;
  if ((err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return err;
  const long long tiles = static_cast<long long>(params.q_blocks) * params.heads;
  if (tiles <= 0 || tiles > (1LL << 30)) return cudaErrorInvalidValue;
  FineBwdParams launch = params;
  if ((err = acquire_tile_counter(stream, &launch.tile_counter)) != cudaSuccess) return err;
  const unsigned grid = static_cast<unsigned>(tiles < sms ? tiles : sms);
  fine_bwd_dq_kernel<<<grid, kThreads, smem, stream>>>(launch);
  return cudaGetLastError();
}

}  // namespace vsa
