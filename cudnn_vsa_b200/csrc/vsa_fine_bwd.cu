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
// left alone.  The FP32 read-modify-write fetches a batch of old values before it stores any, so
// the loads are in flight together.
VSA_DEVICE void store_grad_tile(bool have_acc, uint32_t tmem_addr, float term, uint8_t* turn, int barrier_id, int t,
                                const long long* out_rows, long long out_limit, __nv_bfloat16* out,
                                long long out_row_stride, long long head_offset, float* out_f32, bool accumulate,
                                long long block, long long width, long long head_col, int valid, int computed) {
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
  named_barrier(barrier_id, 128);
  if (f32_out) {
    const float4* rows = reinterpret_cast<const float4*>(turn);  // 32 vectors per row
    float4* base = reinterpret_cast<float4*>(out_f32 + block * kBlock * width + head_col);
    const long long row_vecs = width / 4;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (half * 32 >= valid) break;
      float4 old[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int v = t + (half * 8 + j) * 128, r = v >> 5, c = v & 31;
        old[j] = (accumulate && r < valid) ? base[r * row_vecs + c] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int v = t + (half * 8 + j) * 128, r = v >> 5, c = v & 31;
        if (r < valid) {
          const float4 x = rows[v];
          base[r * row_vecs + c] = make_float4(old[j].x + x.x, old[j].y + x.y, old[j].z + x.z, old[j].w + x.w);
        }
      }
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
  long long out_row[kBlock];
  uint64_t kv_full, q_full[2], do_full[2], q_free[2], do_free[2], sp_done[2], sp_free[2], pd_ready[2], pd_free[2], dkv_final;
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

// One CTA owns one (KV block, head) and walks the query blocks that list it two at a time ("a
// pair", 128 query rows on the M axis): S = Q K^T and dP = dO V^T with M = 128, N = 64, then
// dV^T += dO^T P and dK^T += Q^T dS with the head dims on the M axis and the pair's 128 query
// rows as K.  Query rows sit on the TMEM lanes, so a score-math thread owns one query row and
// needs one LSE and one delta per pair.  Two warpgroups take alternate pairs, each with its own
// S / dP accumulators and P / dS buffers.  A pair's Q stage is held until its dK product has
// read it and its dO stage until the dV product; there is room for two stages of each.  One
// warp issues the score products and another the gradient products, synchronised only through
// mbarriers, so a score product waiting for its refill never holds up a gradient product; Q
// and dO have a producer warp each so that neither load queues behind the other's wait.
__global__ void __launch_bounds__(kDkvThreads, 1) fine_bwd_dkv_kernel(const __grid_constant__ FineBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  DkvSmem& sm = *reinterpret_cast<DkvSmem*>(smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // CTA order: the `first_kv_blocks` leading KV blocks of every head, then the rest head by head.
  int kvb, head;
  {
    const long long id = blockIdx.x, first = p.first_kv_blocks, early = first * p.heads;
    if (id < early) {
      head = static_cast<int>(id / first);
      kvb = static_cast<int>(id - head * first);
    } else {
      const long long rest = p.kv_blocks - first, at = id - early;
      head = static_cast<int>(at / rest);
      kvb = static_cast<int>(first + (at - head * rest));
    }
  }
  const int group = (warp >> 2) & 1;  // score-math warpgroup (warps 0..7 only)
  const int qrow = tid & 127;         // query row of the pair owned by this thread (math role) / head dim (epilogue)
  const uint32_t* mask = p.kv_mask + (static_cast<long long>(head) * p.kv_blocks + kvb) * p.mask_words;
  // Listed query blocks of this tile: every warp counts the row's bits, a few words per lane.
  int n = 0;
  for (int w = p.mask_word_begin + lane; w < p.mask_word_end; w += 32) n += __popc(mask[w]);
#pragma unroll
  for (int shift = 16; shift > 0; shift >>= 1) n += __shfl_xor_sync(0xffffffffu, n, shift);

  if (tid == 0) {
    mbar_init(&sm.kv_full, 1);
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
    sm.abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&p.k_map);
    tma_prefetch_desc(&p.v_map);
    tma_prefetch_desc(&p.q_half_map);
    tma_prefetch_desc(&p.do_half_map);
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
  MaskCursor cursor(mask, p.mask_word_begin, p.mask_word_end);
  const int kv_size = p.kv_sizes != nullptr ? p.kv_sizes[kvb] : kBlock;
  // Keys the products cover: the block's valid keys rounded up to the MMA's N granularity.  A
  // short block (an edge tile of 8, 12, 16 ... keys) runs every product with a narrow N, moves a
  // fraction of the P / dS bytes and does a fraction of the exponentials.
  const int kv_n = kv_size >= kBlock ? kBlock : (kv_size <= 16 ? 16 : ((kv_size + 15) & ~15));

  // Barrier discipline: a barrier is only ever waited on for its NEWEST commit or arrival round;
  // every barrier belongs to one buffer (stage = warpgroup = pair parity) and the round after the
  // awaited one cannot start before the waiter has moved on.
  const int pairs = (n + 1) >> 1;
  if (warp == 9 || warp == 10) {
    // ------------------------------------------------------------ producers: TMA loads
    if (lane == 0 && n > 0) {
      const bool is_q = warp == 9;
      if (is_q) {
        mbar_expect_tx(&sm.kv_full, 2 * kTileBytes);
        tma_load_tile(sm.k, &p.k_map, &sm.kv_full, head, kvb);
        tma_load_tile(sm.v, &p.v_map, &sm.kv_full, head, kvb);
      }
      const CUtensorMap* map = is_q ? &p.q_half_map : &p.do_half_map;
      for (int i = 0; i < pairs; ++i) {
        const int stage = i & 1, count = (2 * i + 1 < n) ? 2 : 1;
        uint64_t* full = is_q ? &sm.q_full[stage] : &sm.do_full[stage];
        uint8_t* dst = is_q ? sm.q[stage] : sm.d_o[stage];
        // The stage was last read by a gradient product of pair i - 2.
        if (i >= 2) mbar_wait(is_q ? &sm.q_free[stage] : &sm.do_free[stage], ((i >> 1) - 1) & 1, abort_flag, p.status, 25);
        mbar_expect_tx(full, count * kTileBytes);
        for (int t = 0; t < count; ++t) {
          const int q_block = cursor.next();
          for (int h = 0; h < 2; ++h) tma_load_half(dst + h * kTileBytes + t * kHalfTileBytes, map, full, head, q_block, h);
        }
      }
    }
  } else if (warp == 11) {
    // ------------------------------------------------------------ issuer of the score products
    // Two issuing warps, one per kind of product, synchronised only through the barriers: the
    // score products of pair j + 2 start as soon as their stage has been refilled and warpgroup
    // j & 1 has pulled pair j out of the accumulators; the gradient products never wait for a
    // refill.  The whole warp walks the loop (uniform control flow and addresses); one elected
    // lane issues the MMAs and commits.
    if (n > 0) {
      const bool leader = elect_one();
      const uint32_t k_lo = umma_desc_lo(smem_u32(sm.k), 16), v_lo = umma_desc_lo(smem_u32(sm.v), 16);
      const uint32_t q_lo0 = umma_desc_lo(smem_u32(sm.q[0]), 16), do_lo0 = umma_desc_lo(smem_u32(sm.d_o[0]), 16);
      constexpr uint32_t kPairLo = kPairBytes >> 4;
      const uint32_t idesc = umma_idesc(128, kv_n, 0, 0);
      mbar_wait(&sm.kv_full, 0, abort_flag, p.status, 21);
      for (int j = 0; j < pairs; ++j) {
        const int b = j & 1;
        if (j >= 2) mbar_wait(&sm.sp_free[b], ((j >> 1) - 1) & 1, abort_flag, p.status, 28);
        mbar_wait(&sm.q_full[b], (j >> 1) & 1, abort_flag, p.status, 26);
        tc_fence_after();
        if (leader) issue_pair_scores(tmem + b * 128, q_lo0 + b * kPairLo, k_lo, idesc);
        mbar_wait(&sm.do_full[b], (j >> 1) & 1, abort_flag, p.status, 30);
        tc_fence_after();
        if (leader) {
          issue_pair_scores(tmem + b * 128 + 64, do_lo0 + b * kPairLo, v_lo, idesc);
          umma_commit(&sm.sp_done[b]);
        }
      }
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------ issuer of the gradient products
    if (n > 0) {
      const bool leader = elect_one();
      const uint32_t q_mn_lo0 = umma_desc_lo(smem_u32(sm.q[0]), kTileBytes);
      const uint32_t do_mn_lo0 = umma_desc_lo(smem_u32(sm.d_o[0]), kTileBytes);
      const uint32_t pt_lo0 = umma_desc_lo(smem_u32(sm.pt[0]), kHalfTileBytes);
      const uint32_t dst_lo0 = umma_desc_lo(smem_u32(sm.dst[0]), kHalfTileBytes);
      constexpr uint32_t kPairLo = kPairBytes >> 4, kBufLo = kTileBytes >> 4;
      const uint32_t idesc = umma_idesc(128, kv_n, 1, 1);
      for (int j = 0; j < pairs; ++j) {
        const int b = j & 1;
        mbar_wait(&sm.pd_ready[b], (j >> 1) & 1, abort_flag, p.status, 29);
        tc_fence_after();
        const bool two = 2 * j + 1 < n;
        if (leader) {
          issue_pair_grad(tmem + kColDk, q_mn_lo0 + b * kPairLo, dst_lo0 + b * kBufLo, two, j > 0, idesc);  // dK^T += Q^T dS
          umma_commit(&sm.q_free[b]);
          issue_pair_grad(tmem + kColDv, do_mn_lo0 + b * kPairLo, pt_lo0 + b * kBufLo, two, j > 0, idesc);  // dV^T += dO^T P
          umma_commit(&sm.do_free[b]);
          umma_commit(&sm.pd_free[b]);
        }
      }
      if (leader) umma_commit(&sm.dkv_final);
    }
  } else {
    // ------------------------------------------------------------ score math warpgroups
    const uint32_t tmem_s = tmem + lane_base + group * 128;
    uint8_t* p_row = sm.pt[group] + qrow * 128;
    uint8_t* ds_row = sm.dst[group] + qrow * 128;
    const int tile = qrow >> 6;
    const float scale = p.scale, sl2 = p.scale * kLog2eBwd;
    const long long head_stats = static_cast<long long>(head) * p.q_slots + (qrow & 63);
    // LSE and delta of this thread's query row, fetched one round ahead.  The cursor yields the
    // query blocks in list order: two per pair, and every other pair belongs to this warpgroup.
    float lse_next = -INFINITY, delta_next = 0.f;
    auto fetch = [&](int i) {
      const int q0 = cursor.next(), q1 = cursor.next();
      if (2 * i + tile < n) {
        const long long at = head_stats + static_cast<long long>(tile ? q1 : q0) * kBlock;
        lse_next = p.lse[at];
        delta_next = p.delta[at];
      } else {
        lse_next = -INFINITY;
      }
    };
    if (group == 1) {
      cursor.next();
      cursor.next();
    }
    if (group < pairs) fetch(group);
    for (int i = group; i < pairs; i += 2) {
      const bool live = (2 * i + tile < n) && lse_next != -INFINITY;
      const float neg_lse2 = -lse_next * kLog2eBwd, delta = delta_next;
      if (i + 2 < pairs) {
        cursor.next();
        cursor.next();
        fetch(i + 2);
      }
      mbar_wait(&sm.sp_done[group], (i >> 1) & 1, abort_flag, p.status, 23);
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
        if (c == 0 && i >= 2) mbar_wait(&sm.pd_free[group], ((i >> 1) - 1) & 1, abort_flag, p.status, 24);
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
  }

  // ---------------------------------------------------------------- epilogue
  if (warp < 8) {
    if (n > 0) {
      mbar_wait(&sm.dkv_final, 0, abort_flag, p.status, 27);
      tc_fence_after();
    }
    // Thread = head dim `qrow`; warpgroup 0 writes dK, warpgroup 1 writes dV, each turning its tile
    // through its own half of the P / dS buffers (idle: every gradient product has completed).
    const long long width = static_cast<long long>(p.heads) * kDim;
    const long long col = static_cast<long long>(head) * kDim + qrow;
    const long long head_col = static_cast<long long>(head) * kDim;
    const long long head_offset = static_cast<long long>(head) * p.out_head_stride;
    // A tile without listed query blocks adds nothing to a running FP32 sum.
    const bool nothing = n == 0 && p.f32_accumulate != 0 && p.dk_f32 != nullptr && p.dk_pool == nullptr &&
                         p.dv_pool == nullptr;
    if (nothing) {
    } else if (group == 0) {
      const float term = pool_term(p.dk_pool, p.pool_f32, p.kv_block_coarse, kvb, kv_size, width, col);
      store_grad_tile(n > 0, tmem + lane_base + kColDk, term, sm.pt[0], 2, qrow, sm.out_row, p.kv_out_rows, p.dk,
                      p.out_row_stride, head_offset, p.dk_f32, p.f32_accumulate != 0, kvb, width, head_col, kv_size, kv_n);
    } else {
      const float term = pool_term(p.dv_pool, p.pool_f32, p.kv_block_coarse, kvb, kv_size, width, col);
      store_grad_tile(n > 0, tmem + lane_base + kColDv, term, sm.dst[0], 3, qrow, sm.out_row, p.kv_out_rows, p.dv,
                      p.out_row_stride, head_offset, p.dv_f32, p.f32_accumulate != 0, kvb, width, head_col, kv_size, kv_n);
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
  const long long ctas = static_cast<long long>(params.kv_blocks) * params.heads;
  if (ctas > 0x7fffffffLL) return cudaErrorInvalidValue;
  fine_bwd_dkv_kernel<<<static_cast<unsigned>(ctas), kDkvThreads, smem, stream>>>(params);
  return cudaGetLastError();
}

}  // namespace vsa
