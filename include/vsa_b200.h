/* C ABI of libvsa_b200.so: the sm_100a kernels behind the packed video-sparse-attention path.
 *
 * Conventions
 *   - Every pointer is a device pointer unless stated; the library never allocates, frees or
 *     synchronises, and launches on the stream it is given (`stream` is a cudaStream_t passed as
 *     void*).  The caller allocates every output and every scratch buffer (sizes below), and the
 *     library keeps no mutable global state - with ONE exception, `vsa_route_static`: it works
 *     in a 16 MiB device array that is part of the library image and caches that array's
 *     address per device on the host.  Its first call on a device may make the CUDA runtime
 *     load the module that holds the array (CUDA loads modules lazily), which reserves the
 *     16 MiB at that moment; make that call during set-up, before any stream capture and before
 *     any region of the program that must not allocate.
 *   - Activations are BF16, row-major `[rows, heads, 128]`; a "slot" tensor holds `blocks * 64`
 *     rows (64 zero-padded slots per block).  `width = heads * 128`.
 *   - Return value: 0 on success, otherwise a VSA_STATUS_* code (a CUDA launch error leaves the
 *     cause in cudaGetLastError).  `status` arguments point to one int32 in device memory that a
 *     kernel sets to 100 + site if one of its bounded waits gave up; the host checks it after the
 *     step and may pass null.
 *   - Each entry point names the reference interface it replaces (file:line in the reference
 *     project).  The reference itself has no native code: these are the calls a maintainer binds
 *     with ctypes in place of the Triton kernels, the cuDNN block-sparse call and the FA4 call.
 */
#ifndef VSA_B200_H_
#define VSA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VSA_STATUS_OK 0
#define VSA_STATUS_BAD_ARGUMENT 1
#define VSA_STATUS_CUDA_ERROR 2
#define VSA_STATUS_NO_DRIVER_ENTRY 3
#define VSA_STATUS_TENSOR_MAP 4
#define VSA_STATUS_TOO_LARGE 5
#define VSA_STATUS_STATIC_SCRATCH 6 /* request does not fit the library's built-in scratch array */

/* Library version, bumped when a signature changes. */
int vsa_abi_version(void);

/* out[i, :] = map[i] >= 0 ? x[map[i], :] : 0 for `out_rows` rows of `row_bytes` bytes.
 * Replaces vsa_kernels.py:66-83 (`gather`, slot padding / restore and their adjoints) and the
 * forward direction of vsa_kernels.py:11-42 (`reorder_tokens`). */
int vsa_row_gather(const void* x, const int64_t* map, void* out, int64_t out_rows, int64_t row_bytes, void* stream);

/* out[rows[i], :] = x[i, :] for `in_rows` unique rows; `out` rows that are not listed keep their
 * content (the caller zero-fills it when the listed rows are a shard).
 * Replaces the inverse direction of vsa_kernels.py:11-42. */
int vsa_row_scatter(const void* x, const int64_t* rows, void* out, int64_t in_rows, int64_t row_bytes, void* stream);

/* Q, K, V rows -> zero-padded slot tensors + FP32 block means (+ BF16 means placed at the
 * block's row of the coarse streams).  `slot_row` null: inputs already are the slots.  Any of
 * `*_slots`, `mean_f32`, `mean_bf16` may be null to skip that output.
 * mean_f32: [3, blocks, width]; mean_bf16: [3, coarse_rows, width] (caller zero-fills it).
 * Replaces vsa_kernels.py:99-101, 119-158 (Q/K/V slot gather) and :161-188 (block means). */
int vsa_slots_pool(const void* q, const void* k, const void* v, const int64_t* slot_row, const int32_t* block_sizes,
                   void* q_slots, void* k_slots, void* v_slots, float* mean_f32, const int32_t* block_coarse,
                   void* mean_bf16, int64_t coarse_rows, int64_t blocks, int32_t heads, void* stream);

/* vsa_slots_pool for q, k, v that are fields of one interleaved tensor, e.g. the caller's fused
 * QKV + gate projection output viewed as [rows, heads, 4, 128]: element (row, head, d) of each
 * input sits at row * in_row_stride + head * in_head_stride + d (in elements, multiples of 8;
 * heads * 128 and 128 describe a contiguous tensor).  The slot tensors and means it writes are
 * contiguous as always.  Relaxes the materialised-input contract of vsa.py:50-61: the
 * `.contiguous()` copies of q, k and v that precede the reference's slot gather disappear. */
int vsa_slots_pool_strided(const void* q, const void* k, const void* v, int64_t in_row_stride, int64_t in_head_stride,
                           const int64_t* slot_row, const int32_t* block_sizes, void* q_slots, void* k_slots,
                           void* v_slots, float* mean_f32, const int32_t* block_coarse, void* mean_bf16,
                           int64_t coarse_rows, int64_t blocks, int32_t heads, void* stream);

/* Bytes of `scratch` that vsa_route needs for a region of `rows` query blocks x `region` KV
 * blocks when it may process `heads` heads at once (it processes fewer per pass if given less). */
int64_t vsa_route_scratch_bytes(int64_t rows, int64_t region, int32_t heads);

/* Top-`keep` selection for one video region: for query blocks [q_begin, q_end) and every head,
 * writes the `keep` KV blocks of [kv_first, kv_last) with the highest FP32 scores
 * q_mean[b + q_mean_offset] . k_mean[j + k_mean_offset], ascending, into
 * indices[head][b][cursor .. cursor + keep).  q_mean / k_mean: FP32 [*, heads, 128].
 * Replaces vsa_core.py:61-72 (`_route_group`: SGEMM + topk + sort). */
int vsa_route(const float* q_mean, const float* k_mean, int32_t heads, int32_t q_begin, int32_t q_end,
              int32_t q_mean_offset, int32_t kv_first, int32_t kv_last, int32_t k_mean_offset, int32_t keep,
              int32_t cursor, int32_t* indices, int64_t index_head_stride, int32_t capacity, void* scratch,
              int64_t scratch_bytes, void* stream);

/* vsa_route without a scratch argument, for callers that may not allocate device memory (a
 * runtime plugin whose enqueue hook must not allocate, a process whose device memory belongs to
 * another framework's pool).  No counterpart in the reference, which allocates freely through
 * PyTorch.  The score matrix lives in a 16 MiB array inside the library's device image, held by
 * every GPU that uses this entry point from its first call on that GPU to process exit (see the
 * conventions above about lazy module loading).  One head's scores,
 * (q_end - q_begin) * (kv_last - kv_first) * 4 bytes, must fit in it, otherwise the call returns
 * VSA_STATUS_STATIC_SCRATCH and does nothing; heads beyond what fits run in further passes.
 * The first call on a device queries the array's address on the host: make it during set-up,
 * before any stream capture begins.  After it, a call allocates and frees nothing.  All calls on
 * a device share the array (it keeps the last call's contents; nothing in it needs clearing
 * because each call writes every score it reads), so calls that overlap on the GPU race - keep
 * them on one stream.  Results are identical to vsa_route. */
int vsa_route_static(const float* q_mean, const float* k_mean, int32_t heads, int32_t q_begin, int32_t q_end,
                     int32_t q_mean_offset, int32_t kv_first, int32_t kv_last, int32_t k_mean_offset, int32_t keep,
                     int32_t cursor, int32_t* indices, int64_t index_head_stride, int32_t capacity, void* stream);

/* Self-test of the bounded waits (no counterpart in the reference): launches one small CTA whose
 * thread 0 waits on an mbarrier that nothing completes, for at most `limit_cycles` SM clocks
 * (1 .. the library's own limit of about one second).  The kernel gives up, writes 177 (100 +
 * the self-test's wait site) to *status if it was 0, and returns; later launches work as usual.
 * Tests use it to check that an expired wait is reported and leaves the context usable. */
int vsa_selftest_wait_timeout(int32_t* status, int64_t limit_cycles, void* stream);

/* Block-sparse attention forward over 64-slot blocks (tcgen05 + TMA).
 *   q [q_blocks*64, heads, 128], k / v [kv_blocks*64, heads, 128] BF16 slot tensors;
 *   indices [heads, q_blocks, capacity] (head stride 0 = one table for all heads), counts alike;
 *   kv_sizes [kv_blocks] valid slots per KV block or null.
 *   o_slots [q_blocks*64, heads, 128] BF16 and lse [heads, q_blocks*64] FP32 (natural log, -inf for
 *   an empty list) are always written.
 *   If `out` is non-null the merged result fine + gate * coarse[block_coarse[block]] is also
 *   written to row slot_row[slot] of out [out_rows, heads, 128] (slot_row null = identity,
 *   block_coarse null or -1 = fine only, gate of such rows is never read).
 * Replaces vsa_core.py:15-20, 33-40 (cuDNN BSA forward), vsa_core.py:87-97 (FA4 coarse, when
 * called on the pooled block tokens), vsa_kernels.py:191-201 and vsa.py:111-117 (restore + merge). */
int vsa_fine_fwd(const void* q, const void* k, const void* v, int64_t q_blocks, int64_t kv_blocks, int32_t heads,
                 const int32_t* indices, const int32_t* counts, int64_t index_head_stride, int64_t count_head_stride,
                 int32_t capacity, const int32_t* kv_sizes, float scale, void* o_slots, float* lse,
                 const int64_t* slot_row, const int32_t* block_coarse, const void* gate, const void* coarse,
                 void* out, int64_t out_rows, int32_t* status, void* stream);

/* vsa_fine_fwd with a strided gate: element (row, head, d) of `gate` sits at
 * row * gate_row_stride + head * gate_head_stride + d (the gate field of an interleaved tensor). */
int vsa_fine_fwd_strided(const void* q, const void* k, const void* v, int64_t q_blocks, int64_t kv_blocks,
                         int32_t heads, const int32_t* indices, const int32_t* counts, int64_t index_head_stride,
                         int64_t count_head_stride, int32_t capacity, const int32_t* kv_sizes, float scale,
                         void* o_slots, float* lse, const int64_t* slot_row, const int32_t* block_coarse,
                         const void* gate, int64_t gate_row_stride, int64_t gate_head_stride, const void* coarse,
                         void* out, int64_t out_rows, int32_t* status, void* stream);

/* Ring step of the forward pass: vsa_fine_fwd on the shard that is here, with the online-softmax
 * merge into the running result done in the kernel's epilogue.  o_running [q_blocks*64, heads, 128]
 * FP32 holds the normalised result of the steps so far (zero before the first) and lse_running
 * [heads, q_blocks*64] their LSE (-inf before the first); both are read and updated in place.  A
 * query block whose list is empty at this step leaves its rows untouched.
 * Replaces vsa_core.py:234-240 (cuDNN BSA forward of the step + `_merge_partial`,
 * vsa_kernels.py:375-397). */
int vsa_fine_fwd_running(const void* q, const void* k, const void* v, int64_t q_blocks, int64_t kv_blocks,
                         int32_t heads, const int32_t* indices, const int32_t* counts, int64_t index_head_stride,
                         int64_t count_head_stride, int32_t capacity, const int32_t* kv_sizes, float scale,
                         float* o_running, float* lse_running, int32_t* status, void* stream);

/* Adjoint of the gate merge fused with the slot gather of dO and with delta = rowsum(dO * O_fine).
 *   grad [rows, width] BF16 in caller order -> grad_slots [blocks*64, width] (null: not wanted),
 *   dgate [rows, width], dcoarse [coarse_rows, width], delta [heads, blocks*64] FP32,
 *   coarse_delta [heads, coarse_rows] FP32 = rowsum(dcoarse * coarse).
 * gate / coarse / block_coarse / dgate / dcoarse / coarse_delta are null for packs without coarse.
 * Replaces vsa_kernels.py:204-246 (`_fine_coarse_gate_add_dgate/_dcoarse`) and the dO slot gather. */
int vsa_merge_bwd(const void* grad, const void* gate, const void* coarse, const void* o_slots, const int64_t* slot_row,
                  const int32_t* block_coarse, void* grad_slots, void* dgate, void* dcoarse, float* delta,
                  float* coarse_delta, int64_t blocks, int64_t coarse_rows, int32_t heads, void* stream);

/* vsa_merge_bwd with strided gate and dgate (both with the same strides: the gate field of an
 * interleaved activation tensor and the same field of its gradient). */
int vsa_merge_bwd_strided(const void* grad, const void* gate, int64_t io_row_stride, int64_t io_head_stride,
                          const void* coarse, const void* o_slots, const int64_t* slot_row,
                          const int32_t* block_coarse, void* grad_slots, void* dgate, void* dcoarse, float* delta,
                          float* coarse_delta, int64_t blocks, int64_t coarse_rows, int32_t heads, void* stream);

/* Words per (head, KV block) row of the query-block bitmask used by vsa_fine_bwd. */
int64_t vsa_kv_mask_words(int64_t q_blocks);

/* Block-sparse attention backward (two tcgen05 kernels, no atomics).
 *   d_o: dO in slot order; lse from the forward; delta = rowsum(dO * O).
 *   kv_mask: scratch of heads * kv_blocks * vsa_kv_mask_words(q_blocks) uint32, rebuilt each call.
 *   BF16 outputs dq [q_out_rows, width], dk / dv [kv_out_rows, width] receive row slot_row[slot]
 *   (null map = identity; padding slots are skipped), plus pool[block] / max(size, 1) when a
 *   pooled-mean gradient is given: pool_f32 = 0 -> BF16 rows indexed by *_block_coarse[block],
 *   pool_f32 = 1 -> FP32 rows indexed by block.
 *   If dq_f32 / dk_f32 / dv_f32 are non-null the results go to those FP32 slot-order buffers
 *   instead (added to their content when f32_accumulate != 0) - the ring path's running dQ and
 *   travelling dK / dV (vsa_kernels.py:356-372).
 *   `parts` selects what runs: bit 0 rebuilds kv_mask, bit 1 the dQ kernel, bit 2 the dK/dV
 *   kernel (7 = everything; the pieces can be launched and timed one by one).  Bits 8-27 hold a
 *   scheduling hint for the dK/dV kernel: that many leading KV blocks (ids 0 .. hint-1) start
 *   before all others for every head.  Pass the number of always-visible blocks at the front of
 *   the KV numbering: every query block lists them, so they run many times longer than the rest
 *   and would otherwise finish last.  The hint changes launch order only, never results.
 * Replaces vsa_core.py:23-30, 42-47 (cuDNN BSA backward), the FA4 backward of the coarse call,
 * the pooling adjoint of vsa_kernels.py:161-176 and the slot->row gathers of :86-96. */
int vsa_fine_bwd(const void* q, const void* k, const void* v, const void* d_o, int64_t q_blocks, int64_t kv_blocks,
                 int32_t heads, const int32_t* indices, const int32_t* counts, int64_t index_head_stride,
                 int64_t count_head_stride, int32_t capacity, const int32_t* q_sizes, const int32_t* kv_sizes,
                 float scale, const float* lse, const float* delta, uint32_t* kv_mask, void* dq, void* dk, void* dv,
                 int64_t q_out_rows, int64_t kv_out_rows, const int64_t* q_slot_row, const int64_t* kv_slot_row,
                 const void* dq_pool, const void* dk_pool, const void* dv_pool, int32_t pool_f32,
                 const int32_t* q_block_coarse, const int32_t* kv_block_coarse, float* dq_f32, float* dk_f32,
                 float* dv_f32, int32_t f32_accumulate, int32_t parts, int32_t* status, void* stream);

/* vsa_fine_bwd writing BF16 dq / dk / dv rows with strides: element (row, head, d) goes to
 * row * out_row_stride + head * out_head_stride + d of each output (the q, k, v fields of the
 * gradient of an interleaved projection output, so no concatenation follows).  BF16 outputs only. */
int vsa_fine_bwd_strided(const void* q, const void* k, const void* v, const void* d_o, int64_t q_blocks,
                         int64_t kv_blocks, int32_t heads, const int32_t* indices, const int32_t* counts,
                         int64_t index_head_stride, int64_t count_head_stride, int32_t capacity,
                         const int32_t* q_sizes, const int32_t* kv_sizes, float scale, const float* lse,
                         const float* delta, uint32_t* kv_mask, void* dq, void* dk, void* dv, int64_t out_row_stride,
                         int64_t out_head_stride, int64_t q_out_rows, int64_t kv_out_rows, const int64_t* q_slot_row,
                         const int64_t* kv_slot_row, const void* dq_pool, const void* dk_pool, const void* dv_pool,
                         int32_t pool_f32, const int32_t* q_block_coarse, const int32_t* kv_block_coarse,
                         int32_t parts, int32_t* status, void* stream);

/* Ring step in passes over sub-ranges of the shard.  A shard whose K and V of one head exceed the
 * L2 cache is walked in `chunks` passes of `chunk_blocks` KV blocks each, so that the CTAs that run
 * together read the same cache-resident part of it; lists are ascending, so the entries of one
 * pass are a contiguous sub-range of every list.
 *   vsa_list_bounds: bounds [rows, chunks + 1] int32; bounds[r][c] = first position of row r whose
 *     block id is >= c * chunk_blocks, bounds[r][chunks] = counts[r].  lists [rows, capacity].
 *   vsa_fine_fwd_running_range: vsa_fine_fwd_running on the entries [b[0], b[1]) of every list, with
 *     b = list_bounds + (head * count_head_stride + block) * bounds_stride (pass `bounds + c` for
 *     pass c and bounds_stride = chunks + 1).
 *   vsa_fine_bwd_range: vsa_fine_bwd with FP32 results only (ring form).  parts & 1 builds the mask
 *     from the whole lists (`counts`); parts & 2 runs the dQ kernel on the list sub-range (null
 *     list_bounds = whole lists); parts & 4 runs the dK/dV kernel over the query blocks of mask
 *     words [mask_word_begin, mask_word_end) only (32 query blocks per word; the passes of one
 *     step add into dk_f32 / dv_f32 with f32_accumulate = 1 after the first).
 * No counterpart in the reference, whose ring step is one cuDNN call per shard (vsa_core.py:234-240). */
int vsa_list_bounds(const int32_t* lists, const int32_t* counts, int64_t rows, int32_t capacity, int32_t chunk_blocks,
                    int32_t chunks, int32_t* bounds, void* stream);
int vsa_fine_fwd_running_range(const void* q, const void* k, const void* v, int64_t q_blocks, int64_t kv_blocks,
                               int32_t heads, const int32_t* indices, const int32_t* list_bounds,
                               int64_t index_head_stride, int64_t count_head_stride, int32_t bounds_stride,
                               int32_t capacity, const int32_t* kv_sizes, float scale, float* o_running,
                               float* lse_running, int32_t* status, void* stream);
int vsa_fine_bwd_range(const void* q, const void* k, const void* v, const void* d_o, int64_t q_blocks,
                       int64_t kv_blocks, int32_t heads, const int32_t* indices, const int32_t* counts,
                       const int32_t* list_bounds, int64_t index_head_stride, int64_t count_head_stride,
                       int32_t bounds_stride, int32_t capacity, const int32_t* q_sizes, const int32_t* kv_sizes,
                       float scale, const float* lse, const float* delta, uint32_t* kv_mask, int32_t mask_word_begin,
                       int32_t mask_word_end, float* dq_f32, float* dk_f32, float* dv_f32, int32_t f32_accumulate,
                       int32_t parts, int32_t* status, void* stream);

/* Ring: split routing rows into per-owner lists of owner-local block ids.
 *   index [rows, capacity], counts [rows], global_to_gather [global blocks] int64.
 *   out_lists [ring_size][list_stride] holds rows of `out_capacity` ids, out_counts
 *   [ring_size][count_stride].  Replaces vsa_kernels.py:285-353 (`partition_indices`). */
int vsa_partition_indices(const int32_t* index, const int32_t* counts, const int64_t* global_to_gather,
                          int32_t* out_lists, int32_t* out_counts, int64_t rows, int32_t capacity,
                          int32_t out_capacity, int32_t ring_size, int32_t peer_blocks, int64_t list_stride,
                          int64_t count_stride, void* stream);

/* Ring: merge one step's normalised partial output (BF16 [slots, heads, 128]) and LSE
 * ([heads, slots]) into the running FP32 output and LSE, in place.
 * Replaces vsa_kernels.py:375-397 (`_merge_partial`). */
int vsa_merge_partial(float* out, float* lse, const void* part, const float* part_lse, int64_t slots, int32_t heads,
                      void* stream);

/* Ring: last step of the forward pass.  fine: running FP32 output in slot order [blocks*64, width];
 * writes its BF16 copy to o_slots (null: not wanted) and out[slot_row[slot]] = fine + gate *
 * coarse[block_coarse[block]] (same rules as the merge epilogue of vsa_fine_fwd).
 * Replaces the `.to(bf16)` of vsa_core.py:243 plus vsa.py:111-117 on the ring path. */
int vsa_gate_merge(const float* fine, const int64_t* slot_row, const int32_t* block_coarse, const void* gate,
                   const void* coarse, void* o_slots, void* out, int64_t blocks, int32_t heads, int64_t out_rows,
                   void* stream);

/* Ring: last step of the backward pass.  acc: FP32 gradient in slot order; writes
 * out[slot_row[slot]] = acc[slot] + pool[row] / max(size, 1) as BF16, where pool is FP32 indexed
 * by block (pool_f32 = 1) or BF16 indexed by block_map[block] (pool_f32 = 0), or null.
 * Replaces the `.to(q.dtype)` of vsa_core.py:285, the pooling adjoint and the slot->row gather. */
int vsa_grad_finish(const float* acc, const int64_t* slot_row, const void* pool, int32_t pool_f32,
                    const int32_t* block_map, const int32_t* block_sizes, void* out, int64_t blocks, int32_t heads,
                    int64_t out_rows, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VSA_B200_H_ */
