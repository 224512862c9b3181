// Shared device helpers for the sm_100a VSA kernels: status codes, bounded mbarrier waits,
// TMA tile loads, tcgen05 (UMMA) descriptors, TMEM allocation and TMEM<->register moves.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vsa {

constexpr int kBlock = 64;   // slots per block
constexpr int kDim = 128;    // head dimension

// Status values returned by the C entry points (0 = success).
enum Status : int {
  kOk = 0,
  kBadArgument = 1,     // null pointer, non-positive size, unsupported width
  kCudaError = 2,       // a CUDA runtime call failed (cudaGetLastError has the cause)
  kNoDriverEntry = 3,   // cuTensorMapEncodeTiled could not be resolved
  kTensorMapError = 4,  // cuTensorMapEncodeTiled rejected the tensor
  kTooLarge = 5,        // size beyond a documented limit
};

// Device-side error word values written through the caller's status pointer.
enum DeviceError : int {
  kDevOk = 0,
  kDevWaitTimeout = 100,  // + a site id: a bounded mbarrier wait gave up
};

#define VSA_DEVICE __device__ __forceinline__

VSA_DEVICE uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------------------------------
// mbarrier
VSA_DEVICE void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
VSA_DEVICE void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
VSA_DEVICE bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Spin limit of every wait in these kernels, in SM clock cycles (about one second).
constexpr long long kWaitCycles = 2000000000LL;

// Bounded wait.  `abort_flag` lives in shared memory; once any wait of the CTA has timed out
// every later wait on an incomplete barrier returns at once, so the CTA drains its loops, frees
// TMEM and exits.  A completed barrier costs one try_wait: the waits of the MMA-issuing thread
// sit on the critical path of the tensor pipe.
VSA_DEVICE bool mbar_wait_limit(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                int site, long long limit_cycles) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_flag) return false;
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - start > limit_cycles) {
      *abort_flag = 1;
      if (status != nullptr) atomicCAS(status, 0, kDevWaitTimeout + site);
      return false;
    }
  }
  return true;
}
VSA_DEVICE bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                          int site) {
  return mbar_wait_limit(bar, parity, abort_flag, status, site, kWaitCycles);
}

// One arrival (release) on an mbarrier whose expected count is the number of arriving threads.
VSA_DEVICE void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Named barrier `id` over `threads` threads (a subset of the CTA's warps).
VSA_DEVICE void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Named barrier that also tells every thread whether `pred` held on all of them.
VSA_DEVICE bool named_barrier_all(int id, int threads, bool pred) {
  uint32_t all;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %3, 0;\n\t"
      "bar.red.and.pred p, %1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(all)
      : "r"(id), "r"(threads), "r"(static_cast<uint32_t>(pred))
      : "memory");
  return all != 0;
}

VSA_DEVICE void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// Make generic-proxy shared-memory writes visible to the async proxy (TMA, tcgen05.mma).
VSA_DEVICE void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Position in a ring of three stages / buffers that keeps counting across tiles: `stage` of the
// next pair, `phase` = parity of that stage's current fill, `round` = fills of stage 0 so far.
struct Ring3 {
  int stage = 0, round = 0;
  uint32_t phase = 0;
  VSA_DEVICE void advance() {
    if (++stage == 3) {
      stage = 0;
      phase ^= 1;
      ++round;
    }
  }
};

// ------------------------------------------------------------------------------------------
// Tile queue of a persistent kernel.  One scheduler thread takes tile numbers (block index first,
// then an atomic counter), looks up what the roles need to know about the tile and publishes it
// in a small ring in shared memory; every other role takes the entries in order.  `count < 0`
// ends the sequence.  Entry `seq` lives in slot seq % kTileRing; its `full` barrier completes
// once per publication, its `free` barrier once all `consumers` have arrived after reading.
constexpr int kTileRing = 4;
struct alignas(16) TileInfo {
  int head, block, count;
  int aux, aux2, aux3;  // kernel-specific (offset into the list, valid rows of the block, its coarse row, ...)
  int reserved[2];
};
struct TileQueue {
  TileInfo info[kTileRing];
  uint64_t full[kTileRing], free_[kTileRing];
};
VSA_DEVICE void tile_queue_init(TileQueue& q, int consumers) {
  for (int i = 0; i < kTileRing; ++i) {
    mbar_init(&q.full[i], 1);
    mbar_init(&q.free_[i], consumers);
  }
}
// Scheduler thread: publish entry `seq`.
VSA_DEVICE void tile_publish(TileQueue& q, int seq, const TileInfo& info, volatile int* abort_flag, int* status,
                             int site) {
  const int slot = seq % kTileRing, round = seq / kTileRing;
  if (round >= 1) mbar_wait(&q.free_[slot], (round - 1) & 1, abort_flag, status, site);
  q.info[slot] = info;
  mbar_arrive(&q.full[slot]);
}
// Any other thread: read entry `seq`.  False when the sequence has ended or a wait gave up.
VSA_DEVICE bool tile_take(TileQueue& q, int seq, TileInfo& info, volatile int* abort_flag, int* status, int site) {
  const int slot = seq % kTileRing;
  const bool ok = mbar_wait(&q.full[slot], (seq / kTileRing) & 1, abort_flag, status, site);
  info = q.info[slot];
  return ok && info.count >= 0;
}
// One arrival per consumer (a warp syncs first, then one lane arrives).
VSA_DEVICE void tile_release(TileQueue& q, int seq) { mbar_arrive(&q.free_[seq % kTileRing]); }

// ------------------------------------------------------------------------------------------
// TMA: the tensor map views a [rows, heads, 128] BF16 tensor as (64 elements, rows, heads, 2 dim
// halves); one box of 64 x 64 x 1 x 2 is a whole 64-row tile, stored [half][row][128 bytes] with
// the 128-byte swizzle.
constexpr int kHalfTileBytes = kBlock * 64 * 2;  // 64 rows x 64 BF16 = 8 KiB
constexpr int kTileBytes = 2 * kHalfTileBytes;   // 64 rows x 128 BF16 = 16 KiB

VSA_DEVICE void tma_load_tile(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int head, int block) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(0),
      "r"(block * kBlock), "r"(head), "r"(0)
      : "memory");
}
// One 64-row x 64-element half of a tile (8 KiB) through a map whose box covers a single half.
VSA_DEVICE void tma_load_half(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int head, int block, int half) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(0),
      "r"(block * kBlock), "r"(head), "r"(half)
      : "memory");
}
VSA_DEVICE void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ------------------------------------------------------------------------------------------
// tcgen05: tensor memory
VSA_DEVICE void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(columns)
               : "memory");
}
VSA_DEVICE void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
VSA_DEVICE void tmem_dealloc(uint32_t base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
VSA_DEVICE void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
VSA_DEVICE void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
VSA_DEVICE void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
VSA_DEVICE void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed.
VSA_DEVICE void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1 (sm_100): 64 bits with
// the start address / 16 in bits 0-13, LBO / 16 in bits 16-29, SBO / 16 in bits 32-45, the version
// in bit 46 and the swizzle mode (2 = 128 bytes) in bits 61-63.
//   K-major operand  (rows = M or N, 128 bytes of K per row): LBO unused, SBO = 1024 (8 rows).
//   MN-major operand (rows = K, 128 bytes of M/N per row): LBO = bytes to the next 64 M/N elements,
//                     SBO = 1024 (next 8 K rows).
// The kernels carry a descriptor as its low word (umma_desc_lo below); the high word is constant.

// Instruction descriptor: BF16 x BF16 -> FP32, dense, M x N, operand majors (0 = K, 1 = MN).
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4)                               // accumulator FP32
         | (1u << 7) | (1u << 10)                // A, B = BF16
         | (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16)
         | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// True in exactly one lane of a converged warp.  Code that the whole warp runs with uniform
// control flow and that only predicates its side effects with this flag keeps its address
// arithmetic warp-uniform, unlike a `lane == 0` branch.
VSA_DEVICE bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// Issue path.  The warp that issues the MMAs has one active lane, so every scalar instruction
// between two MMAs costs its full latency: building two 64-bit descriptors per MMA (about
// twenty dependent instructions) takes longer than the 64 cycles an M64/N128 MMA runs for, and
// the tensor pipe starves.  A descriptor is therefore carried as its low word only (address and
// LBO fields; the operand advances by adding bytes/16), the high word is the constant shared by
// every 128-byte-swizzle operand with SBO = 1024, and the pair is assembled inside the asm.
// D[tmem] (+)= A * B, one K=16 step: `umma_ss_lo` takes both operands from shared memory,
// `umma_ts_lo` takes A from tensor memory (an M x 16 BF16 slice stored like an accumulator of
// the same M, two BF16 per 32-bit column, 8 columns per step).
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO, version 1, SWIZZLE_128B
VSA_DEVICE uint32_t umma_desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
  return ((smem_addr & 0x3FFFF) >> 4) | ((lbo_bytes >> 4) << 16);
}
VSA_DEVICE void umma_ss_lo(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi)
      : "memory");
}
VSA_DEVICE void umma_ts_lo(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi)
      : "memory");
}

// An M=64 accumulator occupies lanes 0..15 of each 32-lane TMEM quarter (row r at lane
// 32*(r/16) + r%16).  The 16x32bx2 shape gives lane t%16 of the warp's quarter to thread t:
// threads 0..15 read columns [col, col+N), threads 16..31 read [col+split, col+split+N).
#define VSA_TMEM_LD_16x32bx2_X32(r, taddr, split)                                                     \
  asm volatile(                                                                                       \
      "tcgen05.ld.sync.aligned.16x32bx2.x32.b32 "                                                     \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                       \
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32], " #split ";" \
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),     \
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),         \
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),      \
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),      \
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])                                                           \
      : "r"(taddr)                                                                                      \
      : "memory")

#define VSA_TMEM_ST_16x32bx2_X32(r, taddr, split)                                                     \
  asm volatile(                                                                                       \
      "tcgen05.st.sync.aligned.16x32bx2.x32.b32 [%0], " #split ", "                                   \
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "                      \
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"              \
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),        \
      "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),       \
      "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),    \
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),    \
      "r"(r[31])                                                                                        \
      : "memory")

#define VSA_TMEM_ST_16x32bx2_X16(r, taddr, split)                                                     \
  asm volatile(                                                                                       \
      "tcgen05.st.sync.aligned.16x32bx2.x16.b32 [%0], " #split ", "                                   \
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"                      \
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),        \
      "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),       \
      "r"(r[15])                                                                                        \
      : "memory")

// An M=128 accumulator has row r in lane r; the 32x32b shape gives lane t of the warp's quarter
// to thread t, with N consecutive columns.
#define VSA_TMEM_LD_32x32b_X32(r, taddr)                                                              \
  asm volatile(                                                                                       \
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                       \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                       \
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"       \
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),     \
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),         \
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),      \
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),      \
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])                                                           \
      : "r"(taddr)                                                                                      \
      : "memory")

// Byte offset of the 16-byte chunk `chunk` (0..7) of row `row` inside a 64-row x 128-byte
// swizzle-128B tile: rows are 128 bytes apart and the chunk index is XORed with row % 8.
VSA_DEVICE uint32_t swizzled_offset(int row, int chunk) {
  return static_cast<uint32_t>(row * 128 + ((chunk ^ (row & 7)) << 4));
}

// Packed FP32 pairs (sm_100 has two-wide FP32 FMA, ADD and MUL): the score-math loops are bound
// by instruction issue, and a packed instruction does the work of two.
using f32x2 = unsigned long long;
VSA_DEVICE f32x2 pack_f32x2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
VSA_DEVICE void unpack_f32x2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
VSA_DEVICE f32x2 fma_f32x2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
VSA_DEVICE f32x2 add_f32x2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
VSA_DEVICE f32x2 mul_f32x2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

VSA_DEVICE uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
VSA_DEVICE float2 unpack_bf16(uint32_t v) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
}

}  // namespace vsa
