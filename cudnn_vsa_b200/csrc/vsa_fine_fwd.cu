// Block-sparse fine attention, forward, for sm_100a.
//
// One CTA owns one (query block, head): 64 query rows against the listed 64-slot KV blocks, taken
// two blocks ("a pair") at a time.  K and V tiles arrive by TMA (128-byte swizzle).  Two tcgen05
// products per pair, both with the 64 query rows as M:
//   S  = Q K^T      N = 128 keys (two KV blocks),  K = 128 head dims   128 accumulator columns
//   O += P V        N = 128 head dims,             K = 128 keys        128 accumulator columns
// The probabilities never touch shared memory: the softmax threads read S from tensor memory,
// write P back as packed BF16 over the first 64 columns of S, and the second product takes P as
// its A operand straight from tensor memory.  The two K tiles of a pair are laid out as one
// 128-row K-major operand ([dim half][tile][row][128 B], four 8 KiB TMA boxes); V tiles stay
// separate and are read MN-major.
//
// S has three buffers in tensor memory (S0 S1 S2 O, 4 x 128 columns, one CTA per SM); one warp
// issues the S products and another the P V products, synchronised only through mbarriers, so
// the softmax of the next pairs runs under the products of their neighbours.  What bounds a pair outside
// the tensor core is the exponential unit (16 per clock per SM: 512 cycles for the 8192 scores
// of a pair), so all 256 softmax threads work on every pair - four threads per query row, 32
// scores each; the two warpgroups exchange the row maxima through shared memory - instead of
// alternating pairs, which would put two pairs' exponentials in flight at once and double the
// latency of each.  (Two independent CTAs per SM fall into lock-step instead: the tensor pipe
// serves their MMAs alternately, both reach their softmax together and the units take turns
// idling.)  The running maximum is raised only when it grew by more than 2^8, and only then do
// the threads of a row rescale that row of O in tensor memory, after the one product that may
// still be accumulating into it has finished.  The epilogue writes the normalised fine output
// in slot order, the natural-log LSE and - when a row map is given - the merged result
// `fine + gate * coarse[block]` straight into the caller's row order, which replaces the
// reference's separate restore and gate-add passes (reference vsa_core.py:15-20,
// vsa_kernels.py:191-201, vsa.py:111-117).  In the ring variant the epilogue instead folds this
// step's partial result into the caller's running FP32 output and LSE (online-softmax merge of
// two normalised partials, reference vsa_kernels.py:375-397 and vsa_core.py:237-240), so a ring
// step neither writes a BF16 partial nor needs a separate merge pass.
//
// The kernel is persistent: one CTA per SM takes (query block, head) tiles in head-major order
// from a work counter (the CTAs of the grid work on neighbouring query blocks of one head at a
// time and share its K / V in L2; lists differ in length, so tiles are handed out as CTAs become
// free rather than dealt in advance).  The thread that loads Q and K is the scheduler: it
// publishes each tile's head, query block and list length (or list sub-range) in a small
// shared-memory queue that the other roles read in order.  Barriers, tensor memory and the
// stage / buffer rings are set up once and simply keep counting across tiles; Q has two buffers,
// so the loads and the first S products of the next tile run under the last softmax rounds and the
// epilogue of the current one.  Two hand-offs exist only between tiles: the S issuer releases a
// Q buffer after the tile's last S product, and the softmax threads release O once the
// epilogue has pulled it out of tensor memory (the next tile's first P V product overwrites it).
#include "vsa_common.cuh"
#include "vsa_kernels.h"

namespace vsa {

namespace {

constexpr int kSoftmaxThreads = 256;  // warps 0..7: softmax and epilogue (four threads per query row)
constexpr int kThreads = 384;         // warp 8: issues the P V products, warp 9: TMA loads of Q and K, warp 10: of V, warp 11: issues the S products
constexpr int kTmemCols = 512;        // S / P buffers b = 0..2 at [128 b, 128 b + 128)   O [384,512)
constexpr int kSBuffers = 3;
constexpr uint32_t kColO = 384;
constexpr int kStages = 3;            // pair stages of K and of V (32 KiB each)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct FwdSmem {  // placed at a 1024-byte aligned address; every tile offset is a multiple of 1024
  uint8_t q[2][kTileBytes];            // Q of the current and of the next tile
  uint8_t k[kStages][2 * kTileBytes];  // [dim half][tile of the pair][row][128 B]
  uint8_t v[kStages][2][kTileBytes];   // [tile of the pair][dim half][row][128 B]
  float m_part[2][2][kBlock];          // [pair parity][warpgroup][query row]: maximum over the warpgroup's columns
  float l_part[2][kBlock];             // [warpgroup][query row]: partial softmax denominators (epilogue)
  // Valid keys of the two KV blocks of a pair (0 = block absent), pair g in slot g % (2 kStages):
  // a slot is rewritten for pair g + 2 kStages only after the S product of pair g + kStages has
  // completed, which needs the P V product - hence the softmax - of pair g.
  int kv_size[2 * kStages][2];
  uint64_t q_full[2], q_free[2], k_full[kStages], v_full[kStages], k_free[kStages], v_free[kStages];
  uint64_t s_done[kSBuffers], p_ready[kSBuffers], p_free[kSBuffers], o_done[2], o_free;
  TileQueue tiles;
  uint32_t tmem_base;
  int abort_flag;
};

VSA_DEVICE float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// S = Q K^T over one or two KV blocks: eight K=16 steps over the two 64-wide dim halves.
// q_lo / k_lo: descriptor low words of the Q tile and of the K pair stage.
VSA_DEVICE void issue_qk(uint32_t tmem_s, uint32_t q_lo, uint32_t k_lo, bool two) {
  const uint32_t idesc = two ? umma_idesc(64, 128, 0, 0) : umma_idesc(64, 64, 0, 0);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    constexpr uint32_t kStep = 32 >> 4;
    umma_ss_lo(tmem_s, q_lo + (ks >> 2) * (kHalfTileBytes >> 4) + (ks & 3) * kStep,
               k_lo + (ks >> 2) * (kTileBytes >> 4) + (ks & 3) * kStep, idesc, ks > 0);
  }
}

// O (+)= P V.  A = P in tensor memory (8 columns per 16 keys); B = V tile [key][dim] read
// MN-major (two 64-wide dim halves 8 KiB apart, 16 keys = 2 KiB per K step).  Only the K=16
// steps that hold valid keys are issued (`steps0` of the first block, `steps1` of the second,
// 0 = block absent): P is zero on masked keys.
VSA_DEVICE void issue_pv(uint32_t tmem_o, uint32_t tmem_p, uint32_t v_lo, int steps0, int steps1, bool accumulate) {
  constexpr uint32_t idesc = umma_idesc(64, 128, 0, 1);
  if (steps0 == 4 && (steps1 == 4 || steps1 == 0)) {
    // Full blocks: straight-line issue, nothing between the MMAs.
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) umma_ts_lo(tmem_o, tmem_p + ks * 8, v_lo + ks * (2048 >> 4), idesc, accumulate || ks > 0);
    if (steps1) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_ts_lo(tmem_o, tmem_p + (4 + ks) * 8, v_lo + (kTileBytes >> 4) + ks * (2048 >> 4), idesc, 1u);
    }
    return;
  }
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
    if (ks < steps0) umma_ts_lo(tmem_o, tmem_p + ks * 8, v_lo + ks * (2048 >> 4), idesc, accumulate || ks > 0);
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
    if (ks < steps1)
      umma_ts_lo(tmem_o, tmem_p + (4 + ks) * 8, v_lo + (kTileBytes >> 4) + ks * (2048 >> 4), idesc, 1u);
}

}  // namespace

// kMode: 0 = fine output and LSE, 1 = also the merged output in the caller's row order,
// 2 = fold the partial result into the running FP32 output and LSE (ring step).
enum : int { kModePlain = 0, kModeMerge = 1, kModeRunning = 2 };

template <int kMode>
__global__ void __launch_bounds__(kThreads, 1) fine_fwd_kernel(const __grid_constant__ FineFwdParams p) {
  constexpr bool kMerge = kMode == kModeMerge;
  extern __shared__ uint8_t smem_raw[];
  FwdSmem& sm = *reinterpret_cast<FwdSmem*>(smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = (warp >> 2) & 1;              // which 32 keys of a KV block (softmax warps 0..7)
  const int row = (warp & 3) * 16 + (lane & 15);  // query row inside the block
  const int half = lane >> 4;                     // which KV block of the pair
  const int tiles = p.q_blocks * p.heads;  // tile t = (head, query block), head-major
  // Consumers of the tile queue: the V producer, the two issuing warps, the eight softmax warps.
  constexpr int kQueueConsumers = 11;
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.q_full[i], 1);
      mbar_init(&sm.q_free[i], 1);
      mbar_init(&sm.o_done[i], 1);
    }
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&sm.k_full[i], 1);
      mbar_init(&sm.v_full[i], 1);
      mbar_init(&sm.k_free[i], 1);
      mbar_init(&sm.v_free[i], 1);
    }
    for (int i = 0; i < kSBuffers; ++i) {
      mbar_init(&sm.s_done[i], 1);
      mbar_init(&sm.p_ready[i], kSoftmaxThreads);
      mbar_init(&sm.p_free[i], 1);
    }
    mbar_init(&sm.o_free, kSoftmaxThreads);
    tile_queue_init(sm.tiles, kQueueConsumers);
    sm.abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&p.q_map);
    tma_prefetch_desc(&p.k_half_map);
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
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  volatile int* abort_flag = &sm.abort_flag;
  const float sl2 = p.scale * kLog2e;
  static_assert(kStages == 3 && kSBuffers == 3, "Ring3 walks the K / V stages and the S buffers");

  // Barrier discipline: a barrier is only ever waited on for its NEWEST commit or arrival round
  // (a wait for an older phase could find the barrier two phases ahead and block).  Every
  // barrier below belongs to one buffer, and the round that follows the awaited one on the same
  // barrier cannot start before the waiter has moved on.  All counters (ring positions, pair
  // parity, number of non-empty tiles) run on across tiles; every role skips empty tiles.
  if (warp == 9) {
    // ------------------------------------------------------------ producer of Q and K
    // K and V have a producer each: their stages are released at different times (K pairs are
    // consumed three pairs ahead of V pairs), and one in-order loop would hold every K load
    // behind the wait for the preceding V stage.
    if (lane == 0) {
      Ring3 ring;
      int slot = 0;       // kv_size slot of the next pair
      int used = 0;       // non-empty tiles so far
      // Tile numbers: the block index first, then the work counter.  The next number is taken
      // only when the last loads of the current tile are about to be issued - a CTA that held
      // tiles in reserve would keep them from idle SMs at the end of the launch, and one list
      // can be a hundred times longer than another - which still leaves the counter and the list
      // length a few pairs of time to arrive.
      auto info_of = [&](int t) -> TileInfo {
        if (t >= tiles) return TileInfo{0, 0, -1};
        const int head = t / p.q_blocks, qb = t - head * p.q_blocks;
        const long long row = static_cast<long long>(head) * p.count_head_stride + qb;
        if (p.list_bounds == nullptr) return TileInfo{head, qb, p.counts[row], 0};
        // aux = first entry of the list's sub-range
        const int32_t* bounds = p.list_bounds + row * p.bounds_stride;
        const int begin = bounds[0];
        return TileInfo{head, qb, bounds[1] - begin, begin};
      };
      auto take_number = [&]() -> int { return static_cast<int>(gridDim.x + atomicAdd(p.tile_counter, 1u)); };
      TileInfo cur = info_of(static_cast<int>(blockIdx.x));
      for (int seq = 0;; ++seq) {
        tile_publish(sm.tiles, seq, cur, abort_flag, p.status, 33);
        if (cur.count < 0 || *abort_flag) break;  // end of the tiles, or a wait gave up: start no further loads
        const int n = cur.count, head = cur.head, qb = cur.block;
        if (n == 0) {
          cur = info_of(take_number());
          continue;
        }
        const int32_t* list = p.indices + static_cast<long long>(head) * p.index_head_stride +
                              static_cast<long long>(qb) * p.capacity + cur.aux;
        const int pairs = (n + 1) >> 1, qbuf = used & 1;
        const int claim_at = pairs > kStages ? pairs - kStages : 0;
        // The Q buffer was last read by the S products of the tile before the previous one.
        if (used >= 2) mbar_wait(&sm.q_free[qbuf], ((used >> 1) - 1) & 1, abort_flag, p.status, 31);
        mbar_expect_tx(&sm.q_full[qbuf], kTileBytes);
        tma_load_tile(sm.q[qbuf], &p.q_map, &sm.q_full[qbuf], head, qb);
        int t_next = tiles;
        for (int i = 0; i < pairs; ++i) {
          if (i == claim_at) t_next = take_number();
          const int count = (2 * i + 1 < n) ? 2 : 1;
          const int stage = ring.stage;
          // The valid length of each block travels with the stage: the softmax threads read it from
          // shared memory after the S product of the stage has completed, instead of chasing
          // list -> sizes through global memory themselves (those loads, queued behind the TMA
          // traffic, cost the softmax loop a tenth of its time).
          const int block0 = list[2 * i], block1 = count == 2 ? list[2 * i + 1] : 0;
          const int size0 = p.kv_sizes != nullptr ? p.kv_sizes[block0] : kBlock;
          const int size1 = count == 2 ? (p.kv_sizes != nullptr ? p.kv_sizes[block1] : kBlock) : 0;
          // Release by the S product of the pair three pairs back.
          if (ring.round >= 1) mbar_wait(&sm.k_free[stage], ring.phase ^ 1, abort_flag, p.status, 3);
          sm.kv_size[slot][0] = size0;
          sm.kv_size[slot][1] = size1;
          mbar_expect_tx(&sm.k_full[stage], count * kTileBytes);
          tma_load_half(sm.k[stage], &p.k_half_map, &sm.k_full[stage], head, block0, 0);
          tma_load_half(sm.k[stage] + kTileBytes, &p.k_half_map, &sm.k_full[stage], head, block0, 1);
          if (count == 2) {
            tma_load_half(sm.k[stage] + kHalfTileBytes, &p.k_half_map, &sm.k_full[stage], head, block1, 0);
            tma_load_half(sm.k[stage] + kTileBytes + kHalfTileBytes, &p.k_half_map, &sm.k_full[stage], head, block1, 1);
          }
          ring.advance();
          if (++slot == 2 * kStages) slot = 0;
        }
        ++used;
        cur = info_of(t_next);
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------ producer of V
    if (lane == 0) {
      Ring3 ring;
      TileInfo info;
      for (int seq = 0; tile_take(sm.tiles, seq, info, abort_flag, p.status, 34); ++seq) {
        tile_release(sm.tiles, seq);
        const int n = info.count, head = info.head, qb = info.block;
        if (n == 0) continue;
        const int32_t* list = p.indices + static_cast<long long>(head) * p.index_head_stride +
                              static_cast<long long>(qb) * p.capacity + info.aux;
        const int pairs = (n + 1) >> 1;
        for (int i = 0; i < pairs; ++i) {
          const int count = (2 * i + 1 < n) ? 2 : 1;
          const int stage = ring.stage;
          if (ring.round >= 1) mbar_wait(&sm.v_free[stage], ring.phase ^ 1, abort_flag, p.status, 10);
          mbar_expect_tx(&sm.v_full[stage], count * kTileBytes);
          for (int u = 0; u < count; ++u) tma_load_tile(sm.v[stage][u], &p.v_map, &sm.v_full[stage], head, list[2 * i + u]);
          ring.advance();
        }
      }
    }
  } else if (warp == 11) {
    // ------------------------------------------------------------ issuer of the S products
    // Two issuing warps, one per kind of product, synchronised only through the barriers, so a
    // wait of one kind never holds up the other.  The whole warp walks the loop (uniform control
    // flow and addresses); one elected lane issues the MMAs and commits.
    const bool leader = elect_one();
    const uint32_t q_lo0 = umma_desc_lo(smem_u32(sm.q[0]), 16);
    const uint32_t k_lo0 = umma_desc_lo(smem_u32(sm.k[0]), 16);
    constexpr uint32_t kStageLo = (2 * kTileBytes) >> 4, kQLo = kTileBytes >> 4;
    Ring3 ring;  // K stage = S buffer of the next S product
    int used = 0;
    TileInfo info;
    for (int seq = 0; __all_sync(0xffffffffu, tile_take(sm.tiles, seq, info, abort_flag, p.status, 35)); ++seq) {
      if (leader) tile_release(sm.tiles, seq);  // after the vote, so every lane has read the entry
      const int n = info.count;
      if (n == 0) continue;
      const int pairs = (n + 1) >> 1, qbuf = used & 1;
      mbar_wait(&sm.q_full[qbuf], (used >> 1) & 1, abort_flag, p.status, 1);
      for (int j = 0; j < pairs; ++j) {
        const int stage = ring.stage;
        // The S product of a pair overwrites P of the pair three back: its P V product must have read it.
        if (ring.round >= 1) mbar_wait(&sm.p_free[stage], ring.phase ^ 1, abort_flag, p.status, 8);
        mbar_wait(&sm.k_full[stage], ring.phase, abort_flag, p.status, 2);
        tc_fence_after();
        if (leader) {
          issue_qk(tmem + stage * 128, q_lo0 + qbuf * kQLo, k_lo0 + stage * kStageLo, 2 * j + 1 < n);
          umma_commit(&sm.s_done[stage]);
          umma_commit(&sm.k_free[stage]);
          if (j + 1 == pairs) umma_commit(&sm.q_free[qbuf]);  // the tile's Q has been read for the last time
        }
        ring.advance();
      }
      ++used;
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------ issuer of the P V products
    const bool leader = elect_one();
    const uint32_t v_lo0 = umma_desc_lo(smem_u32(sm.v[0][0]), kHalfTileBytes);
    constexpr uint32_t kStageLo = (2 * kTileBytes) >> 4;
    Ring3 ring;  // V stage = S / P buffer of the next P V product
    int slot = 0, used = 0;
    uint32_t pair_bit = 0;  // o_done barrier of the next pair
    TileInfo info;
    for (int seq = 0; __all_sync(0xffffffffu, tile_take(sm.tiles, seq, info, abort_flag, p.status, 36)); ++seq) {
      if (leader) tile_release(sm.tiles, seq);
      const int n = info.count;
      if (n == 0) continue;
      const int pairs = (n + 1) >> 1;
      // The first product of a tile overwrites O: the epilogue of the previous tile must have read it.
      if (used >= 1) mbar_wait(&sm.o_free, (used - 1) & 1, abort_flag, p.status, 32);
      for (int i = 0; i < pairs; ++i) {
        const int stage = ring.stage;
        mbar_wait(&sm.p_ready[stage], ring.phase, abort_flag, p.status, 9);
        mbar_wait(&sm.v_full[stage], ring.phase, abort_flag, p.status, 6);
        tc_fence_after();
        // Valid keys of the pair's blocks (written by the K producer with the stage; the softmax
        // that just finished read the same slot).  The first block always gets one step.
        const int size0 = sm.kv_size[slot][0], size1 = sm.kv_size[slot][1];
        const int steps0 = size0 <= 16 ? 1 : (size0 + 15) >> 4, steps1 = (size1 + 15) >> 4;
        if (leader) {
          issue_pv(tmem + kColO, tmem + stage * 128, v_lo0 + stage * kStageLo, steps0, steps1, i > 0);
          umma_commit(&sm.o_done[pair_bit]);
          umma_commit(&sm.v_free[stage]);
          umma_commit(&sm.p_free[stage]);
        }
        ring.advance();
        if (++slot == 2 * kStages) slot = 0;
        pair_bit ^= 1;
      }
      ++used;
    }
  } else {
    // ------------------------------------------------------------ softmax warps and epilogue
    // Thread (row, half, group) owns keys [32 group, 32 group + 32) of KV block `half` of the pair.
    Ring3 ring;           // S buffer of the next pair
    int size_slot = 0;  // kv_size slot of the next pair
    uint32_t pair_bit = 0, pair_round = 0;  // o_done barrier of the next pair / parity of its commit
    TileInfo info;
    // The 256 threads go on only together (they meet at named barriers inside a tile).  The vote
    // also separates the previous epilogue's reads of l_part from this tile's writes.
    for (int seq = 0;
         named_barrier_all(1, kSoftmaxThreads, tile_take(sm.tiles, seq, info, abort_flag, p.status, 37)); ++seq) {
      if (lane == 0) tile_release(sm.tiles, seq);
      const int n = info.count, head = info.head, qb = info.block;
      const int pairs = (n + 1) >> 1;
      float m_ref = -INFINITY;  // running reference maximum of the raw scores of this query row
      float l = 0.f;            // running sum of exp2((s - m_ref) * sl2) over this thread's columns
      uint32_t last_bit = 0, last_round = 0;  // o_done barrier and parity of the tile's last pair
      for (int i = 0; i < pairs; ++i) {
        const int buf = ring.stage;
        const uint32_t tmem_s = tmem + lane_base + buf * 128;
        mbar_wait(&sm.s_done[buf], ring.phase, abort_flag, p.status, 4);
        tc_fence_after();
        // Valid keys among this thread's 32 (the K producer wrote the block sizes with the stage;
        // an odd list ends with half a pair, whose absent block has size 0).
        const int kv_left = sm.kv_size[size_slot][half] - 32 * group;
        uint32_t s_bits[32];
        VSA_TMEM_LD_16x32bx2_X32(s_bits, tmem_s + 32 * group, 64);
        tmem_wait_ld();
        float s[32];
        if (kv_left < 32) {
#pragma unroll
          for (int e = 0; e < 32; ++e) s[e] = e < kv_left ? __uint_as_float(s_bits[e]) : -INFINITY;
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) s[e] = __uint_as_float(s_bits[e]);
        }
        // Four independent chains keep the dependent-latency path short.
        float m4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
        for (int e = 4; e < 32; ++e) m4[e & 3] = fmaxf(m4[e & 3], s[e]);
        float m_pair = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        m_pair = fmaxf(m_pair, __shfl_xor_sync(0xffffffffu, m_pair, 16));
        // The other warpgroup holds the other 64 scores of this row.  Every S read of the pair
        // precedes the barrier, so P may be written over S after it.
        if (half == 0) sm.m_part[pair_bit][group][row] = m_pair;
        named_barrier(1, kSoftmaxThreads);
        m_pair = fmaxf(m_pair, sm.m_part[pair_bit][group ^ 1][row]);
        const float m_new = fmaxf(m_ref, m_pair);
        // Raise the reference maximum only when it moved by more than 2^8; the four threads of a
        // row see the same m_pair, so they decide alike.
        const bool raise = (m_new > m_ref) && (m_ref == -INFINITY || (m_new - m_ref) * sl2 > kRescaleThreshold);
        float alpha = 1.f;
        if (raise) {
          alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2((m_ref - m_new) * sl2);
          m_ref = m_new;
        }
        if (__any_sync(0xffffffffu, raise && i > 0)) {
          // Rare: this thread scales its 32 columns of its row of O, once the P V product of the
          // previous pair - the only one that may still be accumulating - has finished.
          mbar_wait(&sm.o_done[last_bit], last_round, abort_flag, p.status, 5);
          tc_fence_after();
          uint32_t o_bits[32];
          const uint32_t addr = tmem + lane_base + kColO + 32 * group;
          VSA_TMEM_LD_16x32bx2_X32(o_bits, addr, 64);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o_bits[e] = __float_as_uint(__uint_as_float(o_bits[e]) * alpha);
          VSA_TMEM_ST_16x32bx2_X32(o_bits, addr, 64);
        }
        const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref * sl2;
        const f32x2 sl2_2 = pack_f32x2(sl2, sl2), shift_2 = pack_f32x2(-m_use, -m_use);
        uint32_t packed[16];
        f32x2 sum2[4] = {pack_f32x2(0.f, 0.f), pack_f32x2(0.f, 0.f), pack_f32x2(0.f, 0.f), pack_f32x2(0.f, 0.f)};
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float p0, p1;
          unpack_f32x2(fma_f32x2(pack_f32x2(s[e], s[e + 1]), sl2_2, shift_2), p0, p1);
          p0 = fast_exp2(p0);
          p1 = fast_exp2(p1);
          packed[e >> 1] = pack_bf16(p0, p1);
          sum2[(e >> 1) & 3] = add_f32x2(sum2[(e >> 1) & 3], pack_f32x2(p0, p1));
        }
        float lo, hi;
        unpack_f32x2(add_f32x2(add_f32x2(sum2[0], sum2[1]), add_f32x2(sum2[2], sum2[3])), lo, hi);
        l = l * alpha + (lo + hi);
        // P over the first 64 columns of S, two keys per column: block `half` of the pair in
        // columns [32 half, 32 half + 32), this thread's keys in the 16 columns from 16 group.
        VSA_TMEM_ST_16x32bx2_X16(packed, tmem_s + 16 * group, 32);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&sm.p_ready[buf]);
        // This pair's P V product commits to o_done[pair_bit] with parity pair_round.
        last_bit = pair_bit;
        last_round = pair_round;
        ring.advance();
        if (++size_slot == 2 * kStages) size_slot = 0;
        pair_bit ^= 1;
        if (pair_bit == 0) pair_round ^= 1;
      }

      // -------------------------------------------------------------- epilogue of the tile
      if (!(kMode == kModeRunning && n == 0)) {  // an empty ring step leaves the running state as it is
        const long long width = static_cast<long long>(p.heads) * kDim;
        l += __shfl_xor_sync(0xffffffffu, l, 16);
        if (half == 0) sm.l_part[group][row] = l;
        if (n > 0) {
          mbar_wait(&sm.o_done[last_bit], last_round, abort_flag, p.status, 7);
          tc_fence_after();
        }
        named_barrier(1, kSoftmaxThreads);
        const float l_all = sm.l_part[0][row] + sm.l_part[1][row];
        const float inv_l = l_all > 0.f ? 1.f / l_all : 0.f;
        const long long slot = static_cast<long long>(qb) * kBlock + row;
        const float lse_new = l_all > 0.f ? m_ref * p.scale + logf(l_all) : -INFINITY;
        // Thread = (query row, 32 head dims): 64 contiguous bytes of one output row.
        const int dim0 = half * 64 + group * 32;
        const long long col = static_cast<long long>(head) * kDim + dim0;
        uint32_t o_bits[32] = {};
        if (n > 0) {
          VSA_TMEM_LD_16x32bx2_X32(o_bits, tmem + lane_base + kColO + group * 32, 64);
          tmem_wait_ld();
          // O is in registers: the next tile's first P V product may overwrite it.
          tc_fence_before();
          mbar_arrive(&sm.o_free);
        }
        if (kMode == kModeRunning) {
          // running = (running * w_old + partial * w_new) / (w_old + w_new) with LSE weights; rows
          // that have seen no key yet hold LSE = -inf and weight 0.
          float* lse_at = p.lse + static_cast<long long>(head) * p.q_slots + slot;
          const float lse_old = *lse_at;
          float top = fmaxf(lse_old, lse_new);
          if (top == -INFINITY) top = 0.f;
          const float w_old = expf(lse_old - top), w_new = expf(lse_new - top);
          const float denom = w_old + w_new;
          const float inv = denom > 0.f ? 1.f / denom : 0.f;
          const float f_old = w_old * inv, f_new = w_new * inv * inv_l;
          named_barrier(1, kSoftmaxThreads);  // the four threads of a row have read the old LSE
          if (half == 0 && group == 0) *lse_at = top + logf(denom);
          float4* run = reinterpret_cast<float4*>(p.o_running + slot * width + col);
#pragma unroll
          for (int v4 = 0; v4 < 8; ++v4) {
            const float4 old = run[v4];
            float4 r;
            r.x = (w_old > 0.f ? old.x * f_old : 0.f) + __uint_as_float(o_bits[v4 * 4 + 0]) * f_new;
            r.y = (w_old > 0.f ? old.y * f_old : 0.f) + __uint_as_float(o_bits[v4 * 4 + 1]) * f_new;
            r.z = (w_old > 0.f ? old.z * f_old : 0.f) + __uint_as_float(o_bits[v4 * 4 + 2]) * f_new;
            r.w = (w_old > 0.f ? old.w * f_old : 0.f) + __uint_as_float(o_bits[v4 * 4 + 3]) * f_new;
            run[v4] = r;
          }
        } else {
          if (half == 0 && group == 0) p.lse[static_cast<long long>(head) * p.q_slots + slot] = lse_new;
          long long out_row = -1;
          const uint4* gate = nullptr;
          const uint4* coarse = nullptr;
          if (kMerge) {
            out_row = p.slot_row != nullptr ? p.slot_row[slot] : slot;
            if (out_row >= p.out_rows) out_row = -1;
            const int coarse_slot = p.block_coarse != nullptr ? p.block_coarse[qb] : -1;
            if (coarse_slot >= 0 && out_row >= 0) {
              gate = reinterpret_cast<const uint4*>(p.gate + out_row * p.gate_row_stride + head * p.gate_head_stride + dim0);
              coarse = reinterpret_cast<const uint4*>(p.coarse + coarse_slot * width + col);
            }
          }
          uint4* o_dst = reinterpret_cast<uint4*>(p.o_slots + slot * width + col);
          uint4* out_dst = (kMerge && out_row >= 0) ? reinterpret_cast<uint4*>(p.out + out_row * width + col) : nullptr;
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            float o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(o_bits[v4 * 8 + e]) * inv_l;
            o_dst[v4] = make_uint4(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]), pack_bf16(o[4], o[5]), pack_bf16(o[6], o[7]));
            if (kMerge && out_dst != nullptr) {
              if (gate != nullptr) {
                const uint4 g = gate[v4], cz = coarse[v4];
                const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, cw[4] = {cz.x, cz.y, cz.z, cz.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 gf = unpack_bf16(gw[e]), cf = unpack_bf16(cw[e]);
                  // Product and sum are rounded separately, as the reference's merge does.
                  o[2 * e] = __fadd_rn(o[2 * e], __fmul_rn(gf.x, cf.x));
                  o[2 * e + 1] = __fadd_rn(o[2 * e + 1], __fmul_rn(gf.y, cf.y));
                }
              }
              out_dst[v4] = make_uint4(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]), pack_bf16(o[4], o[5]), pack_bf16(o[6], o[7]));
            }
          }
        }
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
  auto kernel = params.o_running != nullptr ? fine_fwd_kernel<kModeRunning>
                                            : (merge ? fine_fwd_kernel<kModeMerge> : fine_fwd_kernel<kModePlain>);
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (err != cudaSuccess) return err;
  // One CTA per SM (a CTA takes a whole SM's shared and tensor memory); fewer when there are fewer tiles.
  int device = 0, sms = 0;
  if ((err = cudaGetDevice(&device)) != cudaSuccess) return err;
  if ((err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return err;
  const long long tiles = static_cast<long long>(params.q_blocks) * params.heads;
  if (tiles <= 0 || tiles > (1LL << 30)) return cudaErrorInvalidValue;
  FineFwdParams launch = params;
  if ((err = acquire_tile_counter(stream, &launch.tile_counter)) != cudaSuccess) return err;
  const unsigned grid = static_cast<unsigned>(tiles < sms ? tiles : sms);
  kernel<<<grid, kThreads, smem, stream>>>(launch);
  return cudaGetLastError();
}

}  // namespace vsa
