// Internal launch interface between the C entry points (vsa_api.cu) and the kernel files.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vsa {

// Zeroed work counter for one persistent kernel launch on `stream` (static device memory of the
// current device; nothing is allocated).
cudaError_t acquire_tile_counter(cudaStream_t stream, unsigned** counter);

// ---------------------------------------------------------------------------- fine attention
struct FineFwdParams {
  CUtensorMap q_map, k_map, v_map;  // [slots, heads, 128] BF16, box 64 x 1 x 64, 128-byte swizzle
  CUtensorMap k_half_map;           // same tensor as k_map, box = one 64-element half of a tile
  const int32_t* indices;           // [heads?, q_blocks, capacity] listed KV blocks, ascending
  const int32_t* counts;            // [heads?, q_blocks]
  long long index_head_stride;      // elements between heads (0 = one table for all heads)
  long long count_head_stride;
  int capacity;
  // Optional sub-range of every list: row r = head * count_head_stride + block uses the entries
  // [list_bounds[r * bounds_stride], list_bounds[r * bounds_stride + 1]) and `counts` is ignored.
  const int32_t* list_bounds;
  int bounds_stride;
  const int32_t* kv_sizes;          // [kv_blocks] valid slots per KV block, or null (all 64)
  __nv_bfloat16* o_slots;           // [q_slots, heads, 128] normalised fine output
  float* lse;                       // [heads, q_slots]
  // Ring step: when set, the partial result is folded into this running FP32 output
  // ([q_slots, heads, 128], normalised) and `lse` is the running LSE, read and updated;
  // o_slots and the merge fields are unused.
  float* o_running;
  // merged output in caller row order (kMerge only)
  const int64_t* slot_row;          // [q_slots] caller row per slot (-1 = padding), null = identity
  const int32_t* block_coarse;      // [q_blocks] coarse row of each query block (-1 = none), or null
  const __nv_bfloat16* gate;        // [out_rows, heads, 128]; element (row, head, d) at row * gate_row_stride + head * gate_head_stride + d
  long long gate_row_stride, gate_head_stride;
  const __nv_bfloat16* coarse;      // [coarse_rows, heads, 128]
  __nv_bfloat16* out;               // [out_rows, heads, 128]
  long long out_rows;
  long long q_slots;
  int q_blocks, heads;
  float scale;
  int* status;
  unsigned* tile_counter;           // set by the launcher
};
cudaError_t launch_fine_fwd(const FineFwdParams& params, bool merge, cudaStream_t stream);

struct FineBwdParams {
  CUtensorMap q_map, k_map, v_map, do_map;  // all [slots, heads, 128] BF16
  CUtensorMap k_half_map, v_half_map;       // same tensors, box = one 64-element half of a tile
  CUtensorMap q_half_map, do_half_map;
  const int32_t* indices;
  const int32_t* counts;
  long long index_head_stride, count_head_stride;
  int capacity;
  // dQ kernel, optional sub-range of every list: row r = head * count_head_stride + block uses the
  // entries [list_bounds[r * bounds_stride], list_bounds[r * bounds_stride + 1]), not `counts`.
  const int32_t* list_bounds;
  int bounds_stride;
  // dK/dV kernel: only the query blocks of mask words [mask_word_begin, mask_word_end) are walked.
  int mask_word_begin, mask_word_end;
  const int32_t* kv_sizes;      // [kv_blocks] or null
  const float* lse;             // [heads, q_slots]
  const float* delta;           // [heads, q_slots] rowsum(dO * O)
  const uint32_t* kv_mask;      // [heads, kv_blocks, mask_words] query blocks that list each KV block
  int mask_words;
  // outputs: gradient rows scattered to caller order, optionally adding the pooled-mean term
  __nv_bfloat16* dq;            // [q_out_rows, heads, 128]
  __nv_bfloat16* dk;            // [kv_out_rows, heads, 128]
  __nv_bfloat16* dv;
  // Element (row, head, d) of dq / dk / dv sits at row * out_row_stride + head * out_head_stride + d
  // (heads * 128 and 128 for contiguous tensors; other values write into an interleaved buffer).
  long long out_row_stride, out_head_stride;
  const int64_t* q_slot_row;    // [q_slots] caller row per slot (-1 = padding) or null (identity)
  const int64_t* kv_slot_row;   // [kv_slots] or null
  // Gradient of the pooled block means, added as pool[block] / max(size, 1) to every valid row.
  // pool_f32 = 0: BF16 rows of the coarse streams, row = *_block_coarse[block] (-1 = none).
  // pool_f32 = 1: FP32 rows indexed by block id (ring: after the reduce-scatter).
  const void* dq_pool;
  const void* dk_pool;
  const void* dv_pool;
  int pool_f32;
  const int32_t* q_block_coarse;
  const int32_t* kv_block_coarse;
  const int32_t* q_sizes;       // [q_blocks] divisor of the pooled term (null = 64)
  // Ring mode: FP32 results in slot order instead of BF16 rows ([slots, heads, 128]); with
  // f32_accumulate the kernel adds to what the buffer holds (running dQ, travelling dK / dV).
  float* dq_f32;
  float* dk_f32;
  float* dv_f32;
  int f32_accumulate;
  // dK/dV kernel: the first `first_kv_blocks` KV blocks are scheduled ahead of all others, for
  // every head (blocks that every query block lists run ten times longer than the rest; started
  // last they would be the tail of the launch).
  int first_kv_blocks;
  long long q_out_rows, kv_out_rows;
  long long q_slots, kv_slots;
  int q_blocks, kv_blocks, heads;
  float scale;
  int* status;
  unsigned* tile_counter;  // set by each launcher
};
cudaError_t launch_fine_bwd_dq(const FineBwdParams& params, cudaStream_t stream);
cudaError_t launch_fine_bwd_dkv(const FineBwdParams& params, cudaStream_t stream);
cudaError_t launch_build_kv_mask(const int32_t* indices, const int32_t* counts, long long index_head_stride,
                                 long long count_head_stride, int capacity, int heads, int q_blocks,
                                 int kv_blocks, uint32_t* mask, int mask_words, cudaStream_t stream);

// ---------------------------------------------------------------------------- row movement
cudaError_t launch_row_gather(const void* x, const int64_t* map, void* out, long long out_rows,
                              long long row_bytes, cudaStream_t stream);
cudaError_t launch_row_scatter(const void* x, const int64_t* rows, void* out, long long in_rows,
                               long long row_bytes, cudaStream_t stream);

// ---------------------------------------------------------------------------- slots + pooling
struct PoolParams {
  const __nv_bfloat16* q;   // [rows, width] caller order (width = heads * 128)
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  // Element (row, head, d) of q / k / v sits at row * in_row_stride + head * in_head_stride + d.
  long long in_row_stride, in_head_stride;
  const int64_t* slot_row;  // [blocks * 64] or null when the inputs already are the slots
  const int32_t* sizes;     // [blocks]
  __nv_bfloat16* q_slots;   // [blocks * 64, width] or null (no slot copy wanted)
  __nv_bfloat16* k_slots;
  __nv_bfloat16* v_slots;
  float* mean_f32;          // [3, blocks, width] FP32 means of q, k, v, or null
  const int32_t* block_coarse;  // [blocks] row of each block in the coarse streams (-1 = none), or null
  __nv_bfloat16* mean_bf16;     // [3, coarse_rows, width] BF16-rounded means at block_coarse rows, or null
  long long coarse_rows;
  long long blocks;
  int width;
};
cudaError_t launch_slots_pool(const PoolParams& params, cudaStream_t stream);

// ---------------------------------------------------------------------------- routing
struct RouteSpan {
  int q_begin, q_end;    // routing rows (query blocks) this span applies to
  int q_mean_offset;     // pooled row of query block b is b + q_mean_offset
  int kv_first, kv_last; // global KV block ids of the video region
  int k_mean_offset;     // pooled row of KV block j is j + k_mean_offset
  int keep;              // blocks to select
  int cursor;            // first column of the routing row to fill
};
// Scores and selection for heads [head0, head0 + head_chunk); `scores` is scratch of at least
// head_chunk * (q_end - q_begin) * (kv_last - kv_first) floats.
cudaError_t launch_route_chunk(const float* q_mean, const float* k_mean, int heads, int head0, int head_chunk,
                               const RouteSpan& span, float* scores, int32_t* indices,
                               long long index_head_stride, int capacity, cudaStream_t stream);

// ---------------------------------------------------------------------------- merge adjoint
struct MergeBwdParams {
  const __nv_bfloat16* grad;     // [rows, width] dO in caller order
  const __nv_bfloat16* gate;     // [rows, width] or null
  // Element (row, head, d) of gate and dgate sits at row * io_row_stride + head * io_head_stride + d.
  long long io_row_stride, io_head_stride;
  const __nv_bfloat16* coarse;   // [coarse_rows, width] or null
  const __nv_bfloat16* o_slots;  // [blocks * 64, width] fine output saved by the forward pass
  const int64_t* slot_row;       // [blocks * 64] or null (identity)
  const int32_t* block_coarse;   // [blocks] or null
  __nv_bfloat16* grad_slots;     // [blocks * 64, width] dO gathered into slots (padding = 0), or null
  __nv_bfloat16* dgate;          // [rows, width] or null
  __nv_bfloat16* dcoarse;        // [coarse_rows, width] or null
  float* delta;                  // [heads, blocks * 64] rowsum(dO * O_fine)
  float* coarse_delta;           // [heads, coarse_rows] rowsum(dcoarse * coarse), or null
  long long blocks;
  long long coarse_rows;
  int heads;
};
cudaError_t launch_merge_bwd(const MergeBwdParams& params, cudaStream_t stream);

// ---------------------------------------------------------------------------- ring helpers
cudaError_t launch_gate_merge(const float* fine, const int64_t* slot_row, const int32_t* block_coarse,
                              const __nv_bfloat16* gate, const __nv_bfloat16* coarse, __nv_bfloat16* o_slots,
                              __nv_bfloat16* out, long long blocks, int heads, long long out_rows,
                              cudaStream_t stream);
cudaError_t launch_grad_finish(const float* acc, const int64_t* slot_row, const void* pool, int pool_f32,
                               const int32_t* block_map, const int32_t* sizes, __nv_bfloat16* out, long long blocks,
                               int heads, long long out_rows, cudaStream_t stream);
cudaError_t launch_partition_indices(const int32_t* index, const int32_t* counts, const int64_t* global_to_gather,
                                     int32_t* out_lists, int32_t* out_counts, long long rows, int capacity,
                                     int out_capacity, int ring_size, int peer_blocks, long long list_stride,
                                     long long count_stride, cudaStream_t stream);
cudaError_t launch_list_bounds(const int32_t* lists, const int32_t* counts, long long rows, int capacity,
                               int chunk_blocks, int chunks, int32_t* bounds, cudaStream_t stream);
cudaError_t launch_merge_partial(float* out, float* lse, const __nv_bfloat16* part, const float* part_lse,
                                 long long slots, int heads, cudaStream_t stream);

}  // namespace vsa
