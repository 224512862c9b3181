// Block-sparse fine attention, backward, for sm_100a: the dK/dV kernel and the bitmask it walks.
// (The dQ kernel lives in vsa_fine_bwd_dq.cu.)  No atomics: the dQ kernel is stationary in the
// query block, this one in the KV block.
//
//   dK/dV kernel  one CTA per (KV block, head), walks the query blocks that list this KV block
//                 (a per-call bitmask built by build_kv_mask_kernel) two at a time:
//                 S = Q K^T, dP = dO V^T, dV^T += dO^T P, dK^T += Q^T dS.
//
// Every product has 128 rows on the M axis (the pair's query rows, or the head dims of the
// transposed gradient accumulators), the shape the tensor core runs at full rate.  P is
// recomputed from the saved LSE (natural log), so no softmax state is carried.  The epilogue
// adds the gradient that reaches a row through its block's pooled mean and scatters the rows
// straight to the caller's row order, skipping padding slots.  Together with the dQ kernel it
// replaces the reference's fine backward call and its slot-to-row gathers
// (reference vsa_core.py:23-30, 42-47; vsa_kernels.py:86-96, 161-176 adjoint).
#include "vsa_common.cuh"
#include "vsa_kernels.h"
#include "vsa_bwd_common.cuh"

namespace vsa {

namespace {

// Epilogue of a transposed accumulator, run by the 128 threads of one warpgroup (`t` = 0..127 =
// TMEM lane = head dim): the columns are the slots of `block`, of which the first `valid` are real
// and the first `computed` (a multiple of 16) were produced by the products.  The tile is turned
// through `turn` (shared memory, 16 KiB for BF16 output, 32 KiB for FP32) so that global memory
// sees 16-byte accesses of whole row segments: `term` is added, then BF16 rows go to the mapped
// rows of `out` (row r, this head at out + row * out_row_stride + head_offset), or FP32 rows in
// slot order to `out_f32` (added to the buffer's content when `accumulate`).  Padding slots are
// left alone.  `release` (or null) gets one arrival per thread once the
// accumulator has been read.
__device__ __noinline__ void store_grad_tile(bool have_acc, uint32_t tmem_addr, float term, uint8_t* turn, int barrier_id, int t,
                                const long long* out_rows, long long out_limit, __nv_bfloat16* out,
                                long long out_row_stride, long long head_offset, float* out_f32, bool accumulate,
                                long long block, long long width, long long head_col, int valid, int computed,
                                uint64_t* release) {
  const bool f32_out = out_f32 != nullptr;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    if (c * 32 >= valid) break;
    uint32_t bits[32] = {};
    if (have_acc && c * 32 < computed) {
      VSA_TMEM_LD_32x32b_X32(bits, tmem_addr + c * 32);
      tmem_wait_ld();
    }
    if (f32_out) {
      float* at = reinterpret_cast<float*>(turn) + c * 32 * kDim + t;
#pragma unroll
      for (int i = 0; i < 32; ++i) at[i * kDim] = __uint_as_float(bits[i]) + term;
    } else {
      __nv_bfloat16* at = reinterpret_cast<__nv_bfloat16*>(turn) + c * 32 * kDim + t;
#pragma unroll
      for (int i = 0; i < 32; ++i) at[i * kDim] = __float2bfloat16(__uint_as_float(bits[i]) + term);
    }
  }
  if (release != nullptr) {
    // The accumulator is in registers / shared memory: the next tile's products may overwrite it.
    tc_fence_before();
    mbar_arrive(release);
  }
  named_barrier(barrier_id, 128);
  if (f32_out) {
    const float4* rows = reinterpret_cast<const float4*>(turn);  // 32 vectors per row
    float4* base = reinterpret_cast<float4*>(out_f32 + block * kBlock * width + head_col);
    const long long row_vecs = width / 4;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int v = t + j * 128, r = v >> 5, c = v & 31;
      if (r >= valid) break;
      // Adding to a running sum is a vector reduction performed by the memory system: nothing is
      // read back, so no load latency sits in the epilogue.  Every element has one writer per
      // launch and launches are ordered by the stream, so the sum is the same as read-add-write.
      if (accumulate)
        atomicAdd(base + r * row_vecs + c, rows[v]);
      else
        base[r * row_vecs + c] = rows[v];
    }
  } else {
    const uint4* rows = reinterpret_cast<const uint4*>(turn);  // 16 vectors per row
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int v = t + j * 128, r = v >> 4, c = v & 15;
      if (r >= valid) break;
      const long long row = out_rows[r];
      if (row >= 0 && row < out_limit) *reinterpret_cast<uint4*>(out + row * out_row_stride + head_offset + c * 8) = rows[v];
    }
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------ dK, dV
namespace {

constexpr int kGroupThreads = 128;  // one score-math warpgroup
constexpr int kDkvThreads = 384;    // warps 0..7: two score-math warpgroups, warp 8: issues the gradient products, warps 9 / 10: TMA loads of K, V, Q / of dO, warp 11: issues the score products
constexpr int kDkvTmemCols = 512;   // per warpgroup g: S [128g, 128g+64)  dP [128g+64, 128g+128);  dK^T [256,320)  dV^T [320,384)
constexpr uint32_t kColDk = 256, kColDv = 320;
constexpr int kPairBytes = 2 * kTileBytes;  // [dim half][tile of the pair][row][128 B]

struct DkvSmem {  // placed at a 1024-byte aligned address; every tile offset is a multiple of 1024
  uint8_t k[kTileBytes];
  uint8_t v[kTileBytes];
  uint8_t q[2][kPairBytes];    // per stage: the Q tiles of two listed query blocks
  uint8_t d_o[2][kPairBytes];
  uint8_t pt[2][kTileBytes];   // per warpgroup: P  [128 queries][64 keys] BF16, 128-byte swizzle
  uint8_t dst[2][kTileBytes];  // per warpgroup: dS [128 queries][64 keys]
  long long out_row[2][kBlock];  // by tile parity
  uint64_t kv_full, kv_free, q_full[2], do_full[2], q_free[2], do_free[2], sp_done[2], sp_free[2], pd_ready[2], pd_free[2];
  uint64_t dkv_final, dkv_free;
  TileQueue tiles;
  uint32_t tmem_base;
  int abort_flag;
};

// Walks the set bits of one (head, KV block) row of the query-block bitmask in ascending order.
// Every thread that needs the sequence keeps its own cursor, so nothing is passed through
// shared memory.
// The two words after the current one are already on their way when the current one runs out, so
// stepping to the next word does not wait for memory (a row has a few set bits per word).
struct MaskCursor {
  const uint32_t* words;  // the whole row
  int end, word;          // walks words [first, end)
  uint32_t bits, ahead1, ahead2;
  VSA_DEVICE MaskCursor() : words(nullptr), end(0), word(0), bits(0u), ahead1(0u), ahead2(0u) {}
  VSA_DEVICE MaskCursor(const uint32_t* w, int first, int e)
      : words(w), end(e), word(first), bits(first < e ? w[first] : 0u), ahead1(first + 1 < e ? w[first + 1] : 0u),
        ahead2(first + 2 < e ? w[first + 2] : 0u) {}
  VSA_DEVICE int next() {
    while (bits == 0) {
      if (++word >= end) return 0;
      bits = ahead1;
      ahead1 = ahead2;
      ahead2 = word + 2 < end ? words[word + 2] : 0u;
    }
    const int bit = __ffs(bits) - 1;
    bits &= bits - 1;
    return word * 32 + bit;
  }
};

// S or dP = A B^T: A = a K-major pair stage (128 query rows), B = the first N rows of the K-major
// K or V tile (N = the block's valid keys rounded up to 16, carried by `idesc`); eight K=16
// steps over the two 64-wide dim halves.
VSA_DEVICE void issue_pair_scores(uint32_t tmem_d, uint32_t pair_lo, uint32_t tile_lo, uint32_t idesc) {
#pragma unroll
  for (int ks = 0; ks < 8; ++ks)
    umma_ss_lo(tmem_d, pair_lo + (ks >> 2) * (kTileBytes >> 4) + (ks & 3) * 2,
               tile_lo + (ks >> 2) * (kHalfTileBytes >> 4) + (ks & 3) * 2, idesc, ks > 0);
}

// D^T[128 dims x N keys] (+)= A^T B over the query rows of one or two blocks: A = a pair stage
// read MN-major (16 rows = 2 KiB per step, dim halves 16 KiB apart), B = the first N keys of the
// P or dS rows [query][key] read MN-major.
VSA_DEVICE void issue_pair_grad(uint32_t tmem_d, uint32_t a_mn_lo, uint32_t b_lo, bool two, bool accumulate,
                                uint32_t idesc) {
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) umma_ss_lo(tmem_d, a_mn_lo + ks * 128, b_lo + ks * 128, idesc, accumulate || ks > 0);
  if (two) {
#pragma unroll
    for (int ks = 4; ks < 8; ++ks) umma_ss_lo(tmem_d, a_mn_lo + ks * 128, b_lo + ks * 128, idesc, 1u);
  }
}

// P and dS of 32 keys of this thread's query row from the S and dP accumulator bits.  kMasked: the
// chunk holds keys at or beyond `kv_size` (padding, or columns the products never wrote), which
// need a select per element; a chunk of valid keys skips it - the math loop is bound by
// instruction issue.  Selects, not products: rows of an absent query block and masked columns may
// hold anything.
template <bool kMasked>
VSA_DEVICE void pds_chunk(const uint32_t (&s_bits)[32], const uint32_t (&dp_bits)[32], bool live, int first_key,
                          int kv_size, float sl2, float neg_lse2, float delta, float scale, uint32_t (&p_packed)[16],
                          uint32_t (&ds_packed)[16]) {
#pragma unroll
  for (int e = 0; e < 32; e += 2) {
    float pr[2], ds[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const bool on = kMasked ? (live && first_key + e + u < kv_size) : live;
      pr[u] = on ? fast_exp2(fmaf(__uint_as_float(s_bits[e + u]), sl2, neg_lse2)) : 0.f;
      ds[u] = on ? pr[u] * (__uint_as_float(dp_bits[e + u]) - delta) * scale : 0.f;
    }
    p_packed[e >> 1] = pack_bf16(pr[0], pr[1]);
    ds_packed[e >> 1] = pack_bf16(ds[0], ds[1]);
  }
}

}  // namespace

// A tile is one (KV block, head): the CTA walks the query blocks that list it two at a time ("a
// pair", 128 query rows on the M axis): S = Q K^T and dP = dO V^T with M = 128, N = 64, then
// dV^T += dO^T P and dK^T += Q^T dS with the head dims on the M axis and the pair's 128 query
// rows as K.  Query rows sit on the TMEM lanes, so a score-math thread owns one query row and
// needs one LSE and one delta per pair.  Two warpgroups take alternate pairs, each with its own
// S / dP accumulators and P / dS buffers.  A pair's Q stage is held until its dK product has
// read it and its dO stage until the dV product; there is room for two stages of each.  One
// warp issues the score products and another the gradient products, synchronised only through
// mbarriers, so a score product waiting for its refill never holds up a gradient product; Q
// and dO have a producer warp each so that neither load queues behind the other's wait.
//
// The kernel is persistent: one CTA per SM takes tiles in launch order (the `first_kv_blocks`
// leading KV blocks of every head, then the rest head by head) from a work counter.  The warp
// that loads K, V and Q is the scheduler: it counts the tile's listed query blocks (the bits of
// its mask row, a few words per lane), looks up the block's valid keys and pooled-gradient row
// and publishes them in a small shared-memory queue that the other roles read in order.
// Barriers, tensor memory and the stage rings are set up once and keep counting across tiles
// (pair g of the CTA uses stage, accumulator set and warpgroup g & 1).  K and V have one buffer:
// the score issuer releases it after the tile's last score products; the math threads release
// the dK^T / dV^T accumulators once the epilogue has read them, and fetch the next tile's output
// rows and first LSE / delta while the epilogue runs.
__global__ void __launch_bounds__(kDkvThreads, 1) fine_bwd_dkv_kernel(const __grid_constant__ FineBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  DkvSmem& sm = *reinterpret_cast<DkvSmem*>(smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = (warp >> 2) & 1;  // score-math warpgroup (warps 0..7 only)
  const int qrow = tid & 127;         // query row of the pair owned by this thread (math role) / head dim (epilogue)
  const int tiles = p.kv_blocks * p.heads;
  // Consumers of the tile queue: the dO producer, the two issuing warps, the eight math warps.
  constexpr int kQueueConsumers = 11;
  // Launch order: the `first_kv_blocks` leading KV blocks of every head, then the rest head by head.
  auto place = [&](int id, int& head, int& kvb) {
    const int first = p.first_kv_blocks, early = first * p.heads;
    if (id < early) {
      head = id / first;
      kvb = id - head * first;
    } else {
      const int rest = p.kv_blocks - first, at = id - early;
      head = at / rest;
      kvb = first + (at - head * rest);
    }
  };
  auto mask_row = [&](int head, int kvb) -> const uint32_t* {
    return p.kv_mask + (static_cast<long long>(head) * p.kv_blocks + kvb) * p.mask_words;
  };
  // Keys the products cover: the block's valid keys rounded up to the MMA's N granularity.  A
  // short block (an edge tile of 8, 12, 16 ... keys) runs every product with a narrow N, moves a
  // fraction of the P / dS bytes and does a fraction of the exponentials.
  auto covered_keys = [](int kv_size) -> int {
    return kv_size >= kBlock ? kBlock : (kv_size <= 16 ? 16 : ((kv_size + 15) & ~15));
  };

  if (tid == 0) {
    mbar_init(&sm.kv_full, 1);
    mbar_init(&sm.kv_free, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.q_full[i], 1);
      mbar_init(&sm.do_full[i], 1);
      mbar_init(&sm.q_free[i], 1);
      mbar_init(&sm.do_free[i], 1);
      mbar_init(&sm.sp_done[i], 1);
      mbar_init(&sm.sp_free[i], kGroupThreads);
      mbar_init(&sm.pd_ready[i], kGroupThreads);
      mbar_init(&sm.pd_free[i], 1);
    }
    mbar_init(&sm.dkv_final, 1);
    mbar_init(&sm.dkv_free, 2 * kGroupThreads);
    tile_queue_init(sm.tiles, kQueueConsumers);
    sm.abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&p.k_map);
    tma_prefetch_desc(&p.v_map);
    tma_prefetch_desc(&p.q_half_map);
    tma_prefetch_desc(&p.do_half_map);
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

  // Barrier discipline: a barrier is only ever waited on for its NEWEST commit or arrival round;
  // every barrier belongs to one buffer (stage = warpgroup = pair parity) and the round after the
  // awaited one cannot start before the waiter has moved on.  Pairs are numbered through all
  // tiles of the CTA (`g`); `used` counts the non-empty tiles so far.  Every role skips empty tiles.
  if (warp == 9) {
    // ------------------------------------------------------------ producer of K, V and Q; scheduler
    // The whole warp walks the tiles (it counts mask bits together); lane 0 issues the loads.
    auto info_of = [&](int t) -> TileInfo {
      if (t >= tiles) return TileInfo{0, 0, -1};
      int head, kvb;
      place(t, head, kvb);
      const uint32_t* mask = mask_row(head, kvb);
      int n = 0;
      for (int w = p.mask_word_begin + lane; w < p.mask_word_end; w += 32) n += __popc(mask[w]);
#pragma unroll
      for (int shift = 16; shift > 0; shift >>= 1) n += __shfl_xor_sync(0xffffffffu, n, shift);
      // aux = valid keys of the block, aux2 = row of its pooled-mean gradients (-1 = none)
      int pool_row = -1;
      if (p.dk_pool != nullptr || p.dv_pool != nullptr)
        pool_row = p.pool_f32 ? kvb : (p.kv_block_coarse != nullptr ? p.kv_block_coarse[kvb] : -1);
      return TileInfo{head, kvb, n, p.kv_sizes != nullptr ? p.kv_sizes[kvb] : kBlock, pool_row};
    };
    int g0 = 0, used = 0;
    TileInfo cur = info_of(static_cast<int>(blockIdx.x));
    for (int seq = 0;; ++seq) {
      if (lane == 0) tile_publish(sm.tiles, seq, cur, abort_flag, p.status, 46);
      // End of the tiles, or a wait gave up: start no further loads.
      if (__any_sync(0xffffffffu, cur.count < 0 || *abort_flag != 0)) break;
      int t_next = tiles;
      if (lane == 0) {
        // The next number is taken only when the last loads of the tile are about to be issued (a CTA
        // that held tiles in reserve would keep them from idle SMs at the end of the launch).
        const int n = cur.count, pairs = (n + 1) >> 1;
        if (n == 0) {
          t_next = static_cast<int>(gridDim.x + atomicAdd(p.tile_counter, 1u));
        } else {
          const int head = cur.head, kvb = cur.block;
          // K and V have one buffer: free once the previous tile's last score products are done.
          if (used >= 1) mbar_wait(&sm.kv_free, (used - 1) & 1, abort_flag, p.status, 52);
          mbar_expect_tx(&sm.kv_full, 2 * kTileBytes);
          tma_load_tile(sm.k, &p.k_map, &sm.kv_full, head, kvb);
          tma_load_tile(sm.v, &p.v_map, &sm.kv_full, head, kvb);
          MaskCursor cursor(mask_row(head, kvb), p.mask_word_begin, p.mask_word_end);
          const int claim_at = pairs > 2 ? pairs - 2 : 0;
          for (int i = 0; i < pairs; ++i) {
            if (i == claim_at) t_next = static_cast<int>(gridDim.x + atomicAdd(p.tile_counter, 1u));
            const int g = g0 + i, stage = g & 1, count = (2 * i + 1 < n) ? 2 : 1;
            // The stage was last read by the dK product of pair g - 2.
            if (g >= 2) mbar_wait(&sm.q_free[stage], ((g >> 1) - 1) & 1, abort_flag, p.status, 25);
            mbar_expect_tx(&sm.q_full[stage], count * kTileBytes);
            for (int t = 0; t < count; ++t) {
              const int q_block = cursor.next();
              for (int h = 0; h < 2; ++h)
                tma_load_half(sm.q[stage] + h * kTileBytes + t * kHalfTileBytes, &p.q_half_map, &sm.q_full[stage], head,
                              q_block, h);
            }
          }
          g0 += pairs;
          ++used;
        }
      }
      t_next = __shfl_sync(0xffffffffu, t_next, 0);
      cur = info_of(t_next);
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------ producer of dO
    if (lane == 0) {
      int g0 = 0;
      TileInfo info;
      for (int seq = 0; tile_take(sm.tiles, seq, info, abort_flag, p.status, 47); ++seq) {
        tile_release(sm.tiles, seq);
        const int n = info.count, pairs = (n + 1) >> 1;
        if (n == 0) continue;
        MaskCursor cursor(mask_row(info.head, info.block), p.mask_word_begin, p.mask_word_end);
        for (int i = 0; i < pairs; ++i) {
          const int g = g0 + i, stage = g & 1, count = (2 * i + 1 < n) ? 2 : 1;
          // The stage was last read by the dV product of pair g - 2.
          if (g >= 2) mbar_wait(&sm.do_free[stage], ((g >> 1) - 1) & 1, abort_flag, p.status, 22);
          mbar_expect_tx(&sm.do_full[stage], count * kTileBytes);
          for (int t = 0; t < count; ++t) {
            const int q_block = cursor.next();
            for (int h = 0; h < 2; ++h)
              tma_load_half(sm.d_o[stage] + h * kTileBytes + t * kHalfTileBytes, &p.do_half_map, &sm.do_full[stage],
                            info.head, q_block, h);
          }
        }
        g0 += pairs;
      }
    }
  } else if (warp == 11) {
    // ------------------------------------------------------------ issuer of the score products
    // Two issuing warps, one per kind of product, synchronised only through the barriers: the
    // score products of pair g + 2 start as soon as their stage has been refilled and warpgroup
    // g & 1 has pulled pair g out of the accumulators; the gradient products never wait for a
    // refill.  The whole warp walks the loop (uniform control flow and addresses); one elected
    // lane issues the MMAs and commits.
    const bool leader = elect_one();
    const uint32_t k_lo = umma_desc_lo(smem_u32(sm.k), 16), v_lo = umma_desc_lo(smem_u32(sm.v), 16);
    const uint32_t q_lo0 = umma_desc_lo(smem_u32(sm.q[0]), 16), do_lo0 = umma_desc_lo(smem_u32(sm.d_o[0]), 16);
    constexpr uint32_t kPairLo = kPairBytes >> 4;
    int g = 0, used = 0;
    TileInfo info;
    for (int seq = 0; __all_sync(0xffffffffu, tile_take(sm.tiles, seq, info, abort_flag, p.status, 48)); ++seq) {
      if (leader) tile_release(sm.tiles, seq);  // after the vote, so every lane has read the entry
      const int n = info.count, pairs = (n + 1) >> 1;
      if (n == 0) continue;
      const uint32_t idesc = umma_idesc(128, covered_keys(info.aux), 0, 0);
      mbar_wait(&sm.kv_full, used & 1, abort_flag, p.status, 21);
      for (int j = 0; j < pairs; ++j, ++g) {
        const int b = g & 1;
        if (g >= 2) mbar_wait(&sm.sp_free[b], ((g >> 1) - 1) & 1, abort_flag, p.status, 28);
        mbar_wait(&sm.q_full[b], (g >> 1) & 1, abort_flag, p.status, 26);
        tc_fence_after();
        if (leader) issue_pair_scores(tmem + b * 128, q_lo0 + b * kPairLo, k_lo, idesc);
        mbar_wait(&sm.do_full[b], (g >> 1) & 1, abort_flag, p.status, 30);
        tc_fence_after();
        if (leader) {
          issue_pair_scores(tmem + b * 128 + 64, do_lo0 + b * kPairLo, v_lo, idesc);
          umma_commit(&sm.sp_done[b]);
          if (j + 1 == pairs) umma_commit(&sm.kv_free);  // K and V have been read for the last time
        }
      }
      ++used;
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------ issuer of the gradient products
    const bool leader = elect_one();
    const uint32_t q_mn_lo0 = umma_desc_lo(smem_u32(sm.q[0]), kTileBytes);
    const uint32_t do_mn_lo0 = umma_desc_lo(smem_u32(sm.d_o[0]), kTileBytes);
    const uint32_t pt_lo0 = umma_desc_lo(smem_u32(sm.pt[0]), kHalfTileBytes);
    const uint32_t dst_lo0 = umma_desc_lo(smem_u32(sm.dst[0]), kHalfTileBytes);
    constexpr uint32_t kPairLo = kPairBytes >> 4, kBufLo = kTileBytes >> 4;
    int g = 0, used = 0;
    TileInfo info;
    for (int seq = 0; __all_sync(0xffffffffu, tile_take(sm.tiles, seq, info, abort_flag, p.status, 49)); ++seq) {
      if (leader) tile_release(sm.tiles, seq);
      const int n = info.count, pairs = (n + 1) >> 1;
      if (n == 0) continue;
      const uint32_t idesc = umma_idesc(128, covered_keys(info.aux), 1, 1);
      // The first products of a tile overwrite dK^T and dV^T: the previous tile's epilogue must have read them.
      if (used >= 1) mbar_wait(&sm.dkv_free, (used - 1) & 1, abort_flag, p.status, 53);
      for (int j = 0; j < pairs; ++j, ++g) {
        const int b = g & 1;
        mbar_wait(&sm.pd_ready[b], (g >> 1) & 1, abort_flag, p.status, 29);
        tc_fence_after();
        const bool two = 2 * j + 1 < n;
        if (leader) {
          issue_pair_grad(tmem + kColDk, q_mn_lo0 + b * kPairLo, dst_lo0 + b * kBufLo, two, j > 0, idesc);  // dK^T += Q^T dS
          umma_commit(&sm.q_free[b]);
          issue_pair_grad(tmem + kColDv, do_mn_lo0 + b * kPairLo, pt_lo0 + b * kBufLo, two, j > 0, idesc);  // dV^T += dO^T P
          umma_commit(&sm.do_free[b]);
          umma_commit(&sm.pd_free[b]);
          if (j + 1 == pairs) umma_commit(&sm.dkv_final);
        }
      }
      ++used;
    }
  } else {
    // ------------------------------------------------------------ score math warpgroups and epilogue
    const uint32_t tmem_s = tmem + lane_base + group * 128;
    uint8_t* p_row = sm.pt[group] + qrow * 128;
    uint8_t* ds_row = sm.dst[group] + qrow * 128;
    const int tile = qrow >> 6;
    const float scale = p.scale, sl2 = p.scale * kLog2eBwd;
    const long long width = static_cast<long long>(p.heads) * kDim;
    // LSE and delta of this thread's query row, fetched one round ahead.  The cursor yields the
    // query blocks in list order: two per pair, and every other pair belongs to this warpgroup.
    MaskCursor cursor;
    float lse_next = -INFINITY, delta_next = 0.f;
    long long pre_row = 0;
    auto fetch = [&](int i, int n, long long head_stats) {
      const int q0 = cursor.next(), q1 = cursor.next();
      if (2 * i + tile < n) {
        const long long at = head_stats + static_cast<long long>(tile ? q1 : q0) * kBlock;
        lse_next = p.lse[at];
        delta_next = p.delta[at];
      } else {
        lse_next = -INFINITY;
      }
    };
    // What a tile needs before its first pair, fetched while the previous tile's epilogue runs: the
    // output row of slot `tid` (threads 0..63), the cursor over its mask row, and LSE / delta of
    // this warpgroup's first pair (`first`, 0 or 1).
    auto start_tile = [&](const TileInfo& t, int first) {
      if (tid < kBlock) {
        const long long s = static_cast<long long>(t.block) * kBlock + tid;
        pre_row = p.kv_slot_row != nullptr ? p.kv_slot_row[s] : s;
      }
      cursor = MaskCursor(mask_row(t.head, t.block), p.mask_word_begin, p.mask_word_end);
      if (first == 1) {
        cursor.next();
        cursor.next();
      }
      lse_next = -INFINITY;
      if (first < ((t.count + 1) >> 1)) fetch(first, t.count, static_cast<long long>(t.head) * p.q_slots + (qrow & 63));
    };

    int g0 = 0;    // pairs of the tiles before the current one
    int used = 0;  // non-empty tiles before the current one
    TileInfo cur;
    // The 256 threads go on only together: they meet at named barriers between tiles.
    bool have = named_barrier_all(1, 2 * kGroupThreads, tile_take(sm.tiles, 0, cur, abort_flag, p.status, 50));
    if (lane == 0) tile_release(sm.tiles, 0);
    if (have) {
      start_tile(cur, group);
      if (tid < kBlock) sm.out_row[0][tid] = pre_row;
      named_barrier(1, 2 * kGroupThreads);
    }
    for (int seq = 0; have; ++seq) {
      const int n = cur.count, head = cur.head, kvb = cur.block, kv_size = cur.aux;
      const int kv_n = covered_keys(kv_size);
      const int pairs = (n + 1) >> 1;
      const long long head_stats = static_cast<long long>(head) * p.q_slots + (qrow & 63);
      // Warpgroup `group` takes the pairs whose running number g0 + i is congruent to it mod 2.
      for (int i = (g0 ^ group) & 1; i < pairs; i += 2) {
        const int g = g0 + i;
        const bool live = (2 * i + tile < n) && lse_next != -INFINITY;
        const float neg_lse2 = -lse_next * kLog2eBwd, delta = delta_next;
        if (i + 2 < pairs) {
          cursor.next();
          cursor.next();
          fetch(i + 2, n, head_stats);
        }
        mbar_wait(&sm.sp_done[group], (g >> 1) & 1, abort_flag, p.status, 23);
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (c * 32 >= kv_n) break;  // a short KV block has no second half
          uint32_t s_bits[32], dp_bits[32];
          VSA_TMEM_LD_32x32b_X32(s_bits, tmem_s + c * 32);
          VSA_TMEM_LD_32x32b_X32(dp_bits, tmem_s + 64 + c * 32);
          tmem_wait_ld();
          if ((c + 1) * 32 >= kv_n) {
            // All of S and dP is in registers: the accumulators may be overwritten.
            tc_fence_before();
            mbar_arrive(&sm.sp_free[group]);
          }
          uint32_t p_packed[16], ds_packed[16];
          if ((c + 1) * 32 <= kv_size)
            pds_chunk<false>(s_bits, dp_bits, live, c * 32, kv_size, sl2, neg_lse2, delta, scale, p_packed, ds_packed);
          else
            pds_chunk<true>(s_bits, dp_bits, live, c * 32, kv_size, sl2, neg_lse2, delta, scale, p_packed, ds_packed);
          // The gradient products of this warpgroup's previous pair have finished reading P / dS.
          if (c == 0 && g >= 2) mbar_wait(&sm.pd_free[group], ((g >> 1) - 1) & 1, abort_flag, p.status, 24);
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            if ((c * 4 + v4) * 8 >= kv_n) break;  // the products read kv_n keys of every row
            const uint32_t off = static_cast<uint32_t>(((c * 4 + v4) ^ (qrow & 7)) << 4);
            *reinterpret_cast<uint4*>(p_row + off) =
                make_uint4(p_packed[4 * v4], p_packed[4 * v4 + 1], p_packed[4 * v4 + 2], p_packed[4 * v4 + 3]);
            *reinterpret_cast<uint4*>(ds_row + off) =
                make_uint4(ds_packed[4 * v4], ds_packed[4 * v4 + 1], ds_packed[4 * v4 + 2], ds_packed[4 * v4 + 3]);
          }
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(&sm.pd_ready[group]);
      }

      // The next tile, and the loads it starts with, under this tile's epilogue.
      TileInfo next;
      const bool have_next =
          named_barrier_all(1, 2 * kGroupThreads, tile_take(sm.tiles, seq + 1, next, abort_flag, p.status, 51));
      if (lane == 0) tile_release(sm.tiles, seq + 1);
      if (have_next) start_tile(next, ((g0 + pairs) ^ group) & 1);

      // -------------------------------------------------------------- epilogue of the tile
      // Thread = head dim `qrow`; warpgroup 0 writes dK, warpgroup 1 writes dV, each turning its tile
      // through half of the P / dS buffers (idle: every gradient product of the tile has completed).
      const long long col = static_cast<long long>(head) * kDim + qrow;
      const long long head_col = static_cast<long long>(head) * kDim;
      const long long head_offset = static_cast<long long>(head) * p.out_head_stride;
      const void* pool = group == 0 ? p.dk_pool : p.dv_pool;
      // Gradient that reaches the rows through the block's pooled mean, already divided by its size.
      float term = 0.f;
      if (pool != nullptr && cur.aux2 >= 0) {
        const long long at = static_cast<long long>(cur.aux2) * width + col;
        term = p.pool_f32 ? static_cast<const float*>(pool)[at]
                          : __bfloat162float(static_cast<const __nv_bfloat16*>(pool)[at]);
        term *= 1.f / static_cast<float>(kv_size > 1 ? kv_size : 1);
      }
      if (n > 0) {
        mbar_wait(&sm.dkv_final, used & 1, abort_flag, p.status, 27);
        tc_fence_after();
      }
      // A tile without listed query blocks adds nothing to a running FP32 sum.
      const bool nothing = n == 0 && p.f32_accumulate != 0 && p.dk_f32 != nullptr && p.dk_pool == nullptr &&
                           p.dv_pool == nullptr;
      uint64_t* release = n > 0 ? &sm.dkv_free : nullptr;
      if (nothing) {
      } else if (group == 0) {
        store_grad_tile(n > 0, tmem + lane_base + kColDk, term, sm.pt[0], 2, qrow, sm.out_row[seq & 1], p.kv_out_rows, p.dk,
                        p.out_row_stride, head_offset, p.dk_f32, p.f32_accumulate != 0, kvb, width, head_col, kv_size, kv_n,
                        release);
      } else {
        store_grad_tile(n > 0, tmem + lane_base + kColDv, term, sm.dst[0], 3, qrow, sm.out_row[seq & 1], p.kv_out_rows, p.dv,
                        p.out_row_stride, head_offset, p.dv_f32, p.f32_accumulate != 0, kvb, width, head_col, kv_size, kv_n,
                        release);
      }
      if (have_next && tid < kBlock) sm.out_row[(seq + 1) & 1][tid] = pre_row;
      // The turning buffers are the next tile's P / dS buffers again, of either warpgroup.
      named_barrier(1, 2 * kGroupThreads);
      g0 += pairs;
      if (n > 0) ++used;
      cur = next;
      have = have_next;
    }
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

cudaError_t launch_fine_bwd_dkv(const FineBwdParams& params, cudaStream_t stream) {
  const size_t smem = sizeof(DkvSmem) + 1024;
  cudaError_t err = cudaFuncSetAttribute(fine_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
  if (err != cudaSuccess) return err;
  // One CTA per SM (a CTA takes a whole SM's shared and tensor memory); fewer when there are fewer tiles.
  int device = 0, sms = 0;
  if ((err = cudaGetDevice(&device)) != cudaSuccess) return err;
  if ((err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return err;
  const long long tiles = static_cast<long long>(params.kv_blocks) * params.heads;
  if (tiles <= 0 || tiles > (1LL << 30)) return cudaErrorInvalidValue;
  FineBwdParams launch = params;
  if ((err = acquire_tile_counter(stream, &launch.tile_counter)) != cudaSuccess) return err;
  const unsigned grid = static_cast<unsigned>(tiles < sms ? tiles : sms);
  fine_bwd_dkv_kernel<<<grid, kDkvThreads, smem, stream>>>(launch);
  return cudaGetLastError();
}

}  // namespace vsa
