// extern "C" entry points of libvsa_b200.so: argument checks, TMA tensor maps, kernel launches.
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/vsa_b200.h"
#include "vsa_common.cuh"
#include "vsa_kernels.h"

namespace {

using vsa::Status;

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is resolved through the runtime, so the library does not link libcuda.
EncodeTiled encode_tiled() {
  static EncodeTiled fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<EncodeTiled>(ptr);
  }();
  return fn;
}

// Tensor map of a BF16 [rows, heads, 128] tensor, described as four dimensions
// (64 elements, rows, heads, 2 halves of the head dim) so that ONE box of 64 x 64 x 1 x 2 brings a
// whole 64-row tile into shared memory as [half][row][128 bytes] with the 128-byte swizzle that
// tcgen05 shared-memory descriptors expect.
int make_tile_map(CUtensorMap* map, const void* base, int64_t rows, int32_t heads, int halves_per_box = 2) {
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return vsa::kNoDriverEntry;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return vsa::kBadArgument;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(heads) * vsa::kDim * 2;
  const cuuint64_t dims[4] = {64, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(heads), 2};
  const cuuint64_t strides[3] = {row_bytes, vsa::kDim * 2, 128};
  const cuuint32_t box[4] = {64, vsa::kBlock, 1, static_cast<cuuint32_t>(halves_per_box)};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  const CUresult res = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box,
                              elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return res == CUDA_SUCCESS ? vsa::kOk : vsa::kTensorMapError;
}

int from_cuda(cudaError_t err) { return err == cudaSuccess ? vsa::kOk : vsa::kCudaError; }
cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

}  // namespace

extern "C" {

int vsa_abi_version(void) { return 1; }

int vsa_row_gather(const void* x, const int64_t* map, void* out, int64_t out_rows, int64_t row_bytes, void* stream) {
  if (out_rows < 0 || row_bytes <= 0) return vsa::kBadArgument;
  if (out_rows == 0) return vsa::kOk;
  if (x == nullptr || map == nullptr || out == nullptr) return vsa::kBadArgument;
  return from_cuda(vsa::launch_row_gather(x, map, out, out_rows, row_bytes, as_stream(stream)));
}

int vsa_row_scatter(const void* x, const int64_t* rows, void* out, int64_t in_rows, int64_t row_bytes, void* stream) {
  if (in_rows < 0 || row_bytes <= 0) return vsa::kBadArgument;
  if (in_rows == 0) return vsa::kOk;
  if (x == nullptr || rows == nullptr || out == nullptr) return vsa::kBadArgument;
  return from_cuda(vsa::launch_row_scatter(x, rows, out, in_rows, row_bytes, as_stream(stream)));
}

}  // extern "C" (reopened below)

namespace {

int slots_pool_common(const void* q, const void* k, const void* v, int64_t in_row_stride, int64_t in_head_stride,
                      const int64_t* slot_row, const int32_t* block_sizes, void* q_slots, void* k_slots,
                      void* v_slots, float* mean_f32, const int32_t* block_coarse, void* mean_bf16,
                      int64_t coarse_rows, int64_t blocks, int32_t heads, void* stream) {
  if (q == nullptr || k == nullptr || v == nullptr || block_sizes == nullptr || blocks < 0 || heads <= 0)
    return vsa::kBadArgument;
  // Rows are read in 16-byte units.
  if (in_row_stride < static_cast<int64_t>(heads) * vsa::kDim || in_head_stride < vsa::kDim ||
      (in_row_stride % 8) != 0 || (in_head_stride % 8) != 0 ||
      ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) != 0)
    return vsa::kBadArgument;
  vsa::PoolParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.in_row_stride = in_row_stride;
  p.in_head_stride = in_head_stride;
  p.slot_row = slot_row;
  p.sizes = block_sizes;
  p.q_slots = static_cast<__nv_bfloat16*>(q_slots);
  p.k_slots = static_cast<__nv_bfloat16*>(k_slots);
  p.v_slots = static_cast<__nv_bfloat16*>(v_slots);
  p.mean_f32 = mean_f32;
  p.block_coarse = block_coarse;
  p.mean_bf16 = static_cast<__nv_bfloat16*>(mean_bf16);
  p.coarse_rows = coarse_rows;
  p.blocks = blocks;
  p.width = heads * vsa::kDim;
  return from_cuda(vsa::launch_slots_pool(p, as_stream(stream)));
}

bool bad_strides(int64_t row_stride, int64_t head_stride, int32_t heads) {
  return row_stride < static_cast<int64_t>(heads) * vsa::kDim || head_stride < vsa::kDim || (row_stride % 8) != 0 ||
         (head_stride % 8) != 0;
}

}  // namespace

extern "C" {

int vsa_slots_pool(const void* q, const void* k, const void* v, const int64_t* slot_row, const int32_t* block_sizes,
                   void* q_slots, void* k_slots, void* v_slots, float* mean_f32, const int32_t* block_coarse,
                   void* mean_bf16, int64_t coarse_rows, int64_t blocks, int32_t heads, void* stream) {
  return slots_pool_common(q, k, v, static_cast<int64_t>(heads) * vsa::kDim, vsa::kDim, slot_row, block_sizes, q_slots,
                           k_slots, v_slots, mean_f32, block_coarse, mean_bf16, coarse_rows, blocks, heads, stream);
}

int vsa_slots_pool_strided(const void* q, const void* k, const void* v, int64_t in_row_stride, int64_t in_head_stride,
                           const int64_t* slot_row, const int32_t* block_sizes, void* q_slots, void* k_slots,
                           void* v_slots, float* mean_f32, const int32_t* block_coarse, void* mean_bf16,
                           int64_t coarse_rows, int64_t blocks, int32_t heads, void* stream) {
  return slots_pool_common(q, k, v, in_row_stride, in_head_stride, slot_row, block_sizes, q_slots, k_slots, v_slots,
                           mean_f32, block_coarse, mean_bf16, coarse_rows, blocks, heads, stream);
}

int64_t vsa_route_scratch_bytes(int64_t rows, int64_t region, int32_t heads) {
  return rows * region * static_cast<int64_t>(heads) * static_cast<int64_t>(sizeof(float));
}

int vsa_route(const float* q_mean, const float* k_mean, int32_t heads, int32_t q_begin, int32_t q_end,
              int32_t q_mean_offset, int32_t kv_first, int32_t kv_last, int32_t k_mean_offset, int32_t keep,
              int32_t cursor, int32_t* indices, int64_t index_head_stride, int32_t capacity, void* scratch,
              int64_t scratch_bytes, void* stream) {
  const int64_t rows = static_cast<int64_t>(q_end) - q_begin, region = static_cast<int64_t>(kv_last) - kv_first;
  if (q_mean == nullptr || k_mean == nullptr || indices == nullptr || heads <= 0 || rows < 0 || region <= 0 ||
      keep < 1 || keep > region || cursor < 0 || cursor + keep > capacity)
    return vsa::kBadArgument;
  if (rows == 0) return vsa::kOk;
  // One score row must fit the select kernel's shared memory.
  if (region * 4 > 200 * 1024) return vsa::kTooLarge;
  const int64_t per_head = rows * region * static_cast<int64_t>(sizeof(float));
  if (scratch == nullptr || scratch_bytes < per_head) return vsa::kBadArgument;
  int64_t chunk = scratch_bytes / per_head;
  if (chunk > heads) chunk = heads;
  const vsa::RouteSpan span{q_begin, q_end, q_mean_offset, kv_first, kv_last, k_mean_offset, keep, cursor};
  for (int32_t head0 = 0; head0 < heads; head0 += static_cast<int32_t>(chunk)) {
    const int32_t now = heads - head0 < chunk ? heads - head0 : static_cast<int32_t>(chunk);
    const cudaError_t err = vsa::launch_route_chunk(q_mean, k_mean, heads, head0, now, span,
                                                    static_cast<float*>(scratch), indices, index_head_stride,
                                                    capacity, as_stream(stream));
    if (err != cudaSuccess) return vsa::kCudaError;
  }
  return vsa::kOk;
}

}  // extern "C" (reopened below)

namespace {

// Shared by the two forward entry points: checks, tensor maps, launch.
int fine_fwd_common(const void* q, const void* k, const void* v, int64_t q_blocks, int64_t kv_blocks, int32_t heads,
                    const int32_t* indices, const int32_t* counts, int64_t index_head_stride,
                    int64_t count_head_stride, int32_t capacity, const int32_t* kv_sizes, float scale, void* o_slots,
                    float* lse, float* o_running, const int64_t* slot_row, const int32_t* block_coarse,
                    const void* gate, int64_t gate_row_stride, int64_t gate_head_stride, const void* coarse,
                    void* out, int64_t out_rows, int32_t* status, void* stream,
                    const int32_t* list_bounds = nullptr, int32_t bounds_stride = 0) {
  if (gate != nullptr && (bad_strides(gate_row_stride, gate_head_stride, heads) ||
                          (reinterpret_cast<uintptr_t>(gate) & 15) != 0))
    return vsa::kBadArgument;
  if (list_bounds != nullptr && bounds_stride < 2) return vsa::kBadArgument;
  if (q == nullptr || k == nullptr || v == nullptr || indices == nullptr ||
      (counts == nullptr && list_bounds == nullptr) ||
      (o_slots == nullptr && o_running == nullptr) || lse == nullptr || q_blocks < 0 || kv_blocks <= 0 ||
      heads <= 0 || capacity <= 0)
    return vsa::kBadArgument;
  if (q_blocks == 0) return vsa::kOk;
  if (q_blocks > 0x7fffffffLL / vsa::kBlock || kv_blocks > 0x7fffffffLL / vsa::kBlock || heads > 65535)
    return vsa::kTooLarge;
  if (block_coarse != nullptr && out != nullptr && (gate == nullptr || coarse == nullptr)) return vsa::kBadArgument;
  if ((reinterpret_cast<uintptr_t>(o_running) & 15) != 0) return vsa::kBadArgument;
  vsa::FineFwdParams p{};
  int rc = make_tile_map(&p.q_map, q, q_blocks * vsa::kBlock, heads);
  if (rc == vsa::kOk) rc = make_tile_map(&p.k_map, k, kv_blocks * vsa::kBlock, heads);
  if (rc == vsa::kOk) rc = make_tile_map(&p.k_half_map, k, kv_blocks * vsa::kBlock, heads, 1);
  if (rc == vsa::kOk) rc = make_tile_map(&p.v_map, v, kv_blocks * vsa::kBlock, heads);
  if (rc != vsa::kOk) return rc;
  p.indices = indices;
  p.counts = counts;
  p.index_head_stride = index_head_stride;
  p.count_head_stride = count_head_stride;
  p.capacity = capacity;
  p.list_bounds = list_bounds;
  p.bounds_stride = bounds_stride;
  p.kv_sizes = kv_sizes;
  p.o_slots = static_cast<__nv_bfloat16*>(o_slots);
  p.lse = lse;
  p.o_running = o_running;
  p.slot_row = slot_row;
  p.block_coarse = block_coarse;
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.gate_row_stride = gate_row_stride;
  p.gate_head_stride = gate_head_stride;
  p.coarse = static_cast<const __nv_bfloat16*>(coarse);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_rows = out_rows;
  p.q_slots = q_blocks * vsa::kBlock;
  p.q_blocks = static_cast<int>(q_blocks);
  p.heads = heads;
  p.scale = scale;
  p.status = status;
  return from_cuda(vsa::launch_fine_fwd(p, out != nullptr, as_stream(stream)));
}

}  // namespace

extern "C" {

int vsa_fine_fwd(const void* q, const void* k, const void* v, int64_t q_blocks, int64_t kv_blocks, int32_t heads,
                 const int32_t* indices, const int32_t* counts, int64_t index_head_stride, int64_t count_head_stride,
                 int32_t capacity, const int32_t* kv_sizes, float scale, void* o_slots, float* lse,
                 const int64_t* slot_row, const int32_t* block_coarse, const void* gate, const void* coarse,
                 void* out, int64_t out_rows, int32_t* status, void* stream) {
  if (o_slots == nullptr) return vsa::kBadArgument;
  return fine_fwd_common(q, k, v, q_blocks, kv_blocks, heads, indices, counts, index_head_stride, count_head_stride,
                         capacity, kv_sizes, scale, o_slots, lse, nullptr, slot_row, block_coarse, gate,
                         static_cast<int64_t>(heads) * vsa::kDim, vsa::kDim, coarse, out, out_rows, status, stream);
}

int vsa_fine_fwd_strided(const void* q, const void* k, const void* v, int64_t q_blocks, int64_t kv_blocks,
                         int32_t heads, const int32_t* indices, const int32_t* counts, int64_t index_head_stride,
                         int64_t count_head_stride, int32_t capacity, const int32_t* kv_sizes, float scale,
                         void* o_slots, float* lse, const int64_t* slot_row, const int32_t* block_coarse,
                         const void* gate, int64_t gate_row_stride, int64_t gate_head_stride, const void* coarse,
                         void* out, int64_t out_rows, int32_t* status, void* stream) {
  if (o_slots == nullptr) return vsa::kBadArgument;
  return fine_fwd_common(q, k, v, q_blocks, kv_blocks, heads, indices, counts, index_head_stride, count_head_stride,
                         capacity, kv_sizes, scale, o_slots, lse, nullptr, slot_row, block_coarse, gate,
                         gate_row_stride, gate_head_stride, coarse, out, out_rows, status, stream);
}

int vsa_fine_fwd_running(const void* q, const void* k, const void* v, int64_t q_blocks, int64_t kv_blocks,
                         int32_t heads, const int32_t* indices, const int32_t* counts, int64_t index_head_stride,
                         int64_t count_head_stride, int32_t capacity, const int32_t* kv_sizes, float scale,
                         float* o_running, float* lse_running, int32_t* status, void* stream) {
  if (o_running == nullptr) return vsa::kBadArgument;
  return fine_fwd_common(q, k, v, q_blocks, kv_blocks, heads, indices, counts, index_head_stride, count_head_stride,
                         capacity, kv_sizes, scale, nullptr, lse_running, o_running, nullptr, nullptr, nullptr, 0, 0,
                         nullptr, nullptr, 0, status, stream);
}

int vsa_fine_fwd_running_range(const void* q, const void* k, const void* v, int64_t q_blocks, int64_t kv_blocks,
                               int32_t heads, const int32_t* indices, const int32_t* list_bounds,
                               int64_t index_head_stride, int64_t count_head_stride, int32_t bounds_stride,
                               int32_t capacity, const int32_t* kv_sizes, float scale, float* o_running,
                               float* lse_running, int32_t* status, void* stream) {
  if (o_running == nullptr || list_bounds == nullptr) return vsa::kBadArgument;
  return fine_fwd_common(q, k, v, q_blocks, kv_blocks, heads, indices, nullptr, index_head_stride, count_head_stride,
                         capacity, kv_sizes, scale, nullptr, lse_running, o_running, nullptr, nullptr, nullptr, 0, 0,
                         nullptr, nullptr, 0, status, stream, list_bounds, bounds_stride);
}

}  // extern "C" (reopened below)

namespace {

int merge_bwd_common(const void* grad, const void* gate, int64_t io_row_stride, int64_t io_head_stride,
                     const void* coarse, const void* o_slots, const int64_t* slot_row, const int32_t* block_coarse,
                     void* grad_slots, void* dgate, void* dcoarse, float* delta, float* coarse_delta, int64_t blocks,
                     int64_t coarse_rows, int32_t heads, void* stream) {
  if (grad == nullptr || o_slots == nullptr || delta == nullptr || blocks < 0 || heads <= 0) return vsa::kBadArgument;
  if (coarse != nullptr && (gate == nullptr || block_coarse == nullptr)) return vsa::kBadArgument;
  if (bad_strides(io_row_stride, io_head_stride, heads) ||
      ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(dgate)) & 15) != 0)
    return vsa::kBadArgument;
  vsa::MergeBwdParams p{};
  p.grad = static_cast<const __nv_bfloat16*>(grad);
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.io_row_stride = io_row_stride;
  p.io_head_stride = io_head_stride;
  p.coarse = static_cast<const __nv_bfloat16*>(coarse);
  p.o_slots = static_cast<const __nv_bfloat16*>(o_slots);
  p.slot_row = slot_row;
  p.block_coarse = block_coarse;
  p.grad_slots = static_cast<__nv_bfloat16*>(grad_slots);
  p.dgate = static_cast<__nv_bfloat16*>(dgate);
  p.dcoarse = static_cast<__nv_bfloat16*>(dcoarse);
  p.delta = delta;
  p.coarse_delta = coarse_delta;
  p.blocks = blocks;
  p.coarse_rows = coarse_rows;
  p.heads = heads;
  return from_cuda(vsa::launch_merge_bwd(p, as_stream(stream)));
}

}  // namespace

extern "C" {

int vsa_merge_bwd(const void* grad, const void* gate, const void* coarse, const void* o_slots, const int64_t* slot_row,
                  const int32_t* block_coarse, void* grad_slots, void* dgate, void* dcoarse, float* delta,
                  float* coarse_delta, int64_t blocks, int64_t coarse_rows, int32_t heads, void* stream) {
  return merge_bwd_common(grad, gate, static_cast<int64_t>(heads) * vsa::kDim, vsa::kDim, coarse, o_slots, slot_row,
                          block_coarse, grad_slots, dgate, dcoarse, delta, coarse_delta, blocks, coarse_rows, heads,
                          stream);
}

int vsa_merge_bwd_strided(const void* grad, const void* gate, int64_t io_row_stride, int64_t io_head_stride,
                          const void* coarse, const void* o_slots, const int64_t* slot_row,
                          const int32_t* block_coarse, void* grad_slots, void* dgate, void* dcoarse, float* delta,
                          float* coarse_delta, int64_t blocks, int64_t coarse_rows, int32_t heads, void* stream) {
  return merge_bwd_common(grad, gate, io_row_stride, io_head_stride, coarse, o_slots, slot_row, block_coarse,
                          grad_slots, dgate, dcoarse, delta, coarse_delta, blocks, coarse_rows, heads, stream);
}

int64_t vsa_kv_mask_words(int64_t q_blocks) { return (q_blocks + 31) / 32; }

}  // extern "C" (reopened below)

namespace {

int fine_bwd_common(const void* q, const void* k, const void* v, const void* d_o, int64_t q_blocks, int64_t kv_blocks,
                    int32_t heads, const int32_t* indices, const int32_t* counts, int64_t index_head_stride,
                    int64_t count_head_stride, int32_t capacity, const int32_t* q_sizes, const int32_t* kv_sizes,
                    float scale, const float* lse, const float* delta, uint32_t* kv_mask, void* dq, void* dk, void* dv,
                    int64_t out_row_stride, int64_t out_head_stride, int64_t q_out_rows, int64_t kv_out_rows,
                    const int64_t* q_slot_row, const int64_t* kv_slot_row, const void* dq_pool, const void* dk_pool,
                    const void* dv_pool, int32_t pool_f32, const int32_t* q_block_coarse,
                    const int32_t* kv_block_coarse, float* dq_f32, float* dk_f32, float* dv_f32,
                    int32_t f32_accumulate, int32_t parts, int32_t* status, void* stream,
                    const int32_t* list_bounds = nullptr, int32_t bounds_stride = 0, int32_t mask_word_begin = 0,
                    int32_t mask_word_end = -1) {
  if (out_row_stride < static_cast<int64_t>(heads) * vsa::kDim || out_head_stride < vsa::kDim) return vsa::kBadArgument;
  if (list_bounds != nullptr && bounds_stride < 2) return vsa::kBadArgument;
  if (q == nullptr || k == nullptr || v == nullptr || d_o == nullptr || indices == nullptr || counts == nullptr ||
      lse == nullptr || delta == nullptr || kv_mask == nullptr || q_blocks <= 0 || kv_blocks <= 0 || heads <= 0 ||
      capacity <= 0)
    return vsa::kBadArgument;
  if (((parts & 2) && dq == nullptr && dq_f32 == nullptr) ||
      ((parts & 4) && ((dk == nullptr && dk_f32 == nullptr) || (dv == nullptr && dv_f32 == nullptr))))
    return vsa::kBadArgument;
  if (q_blocks > 0x7fffffffLL / vsa::kBlock || kv_blocks > 0x7fffffffLL / vsa::kBlock || heads > 65535)
    return vsa::kTooLarge;
  // The LSE / delta rows are fetched with 16-byte bulk copies; the gradients are written with 16-byte stores.
  if (((reinterpret_cast<uintptr_t>(lse) | reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(dq) |
        reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv) | reinterpret_cast<uintptr_t>(dq_f32) |
        reinterpret_cast<uintptr_t>(dk_f32) | reinterpret_cast<uintptr_t>(dv_f32)) & 15) != 0)
    return vsa::kBadArgument;
  vsa::FineBwdParams p{};
  int rc = make_tile_map(&p.q_map, q, q_blocks * vsa::kBlock, heads);
  if (rc == vsa::kOk) rc = make_tile_map(&p.k_map, k, kv_blocks * vsa::kBlock, heads);
  if (rc == vsa::kOk) rc = make_tile_map(&p.v_map, v, kv_blocks * vsa::kBlock, heads);
  if (rc == vsa::kOk) rc = make_tile_map(&p.do_map, d_o, q_blocks * vsa::kBlock, heads);
  if (rc == vsa::kOk) rc = make_tile_map(&p.k_half_map, k, kv_blocks * vsa::kBlock, heads, 1);
  if (rc == vsa::kOk) rc = make_tile_map(&p.v_half_map, v, kv_blocks * vsa::kBlock, heads, 1);
  if (rc == vsa::kOk) rc = make_tile_map(&p.q_half_map, q, q_blocks * vsa::kBlock, heads, 1);
  if (rc == vsa::kOk) rc = make_tile_map(&p.do_half_map, d_o, q_blocks * vsa::kBlock, heads, 1);
  if (rc != vsa::kOk) return rc;
  p.indices = indices;
  p.counts = counts;
  p.index_head_stride = index_head_stride;
  p.count_head_stride = count_head_stride;
  p.capacity = capacity;
  p.kv_sizes = kv_sizes;
  p.lse = lse;
  p.delta = delta;
  p.kv_mask = kv_mask;
  p.mask_words = static_cast<int>(vsa_kv_mask_words(q_blocks));
  p.list_bounds = list_bounds;
  p.bounds_stride = bounds_stride;
  p.mask_word_begin = mask_word_begin;
  p.mask_word_end = mask_word_end < 0 ? p.mask_words : mask_word_end;
  if (p.mask_word_begin < 0 || p.mask_word_end > p.mask_words || p.mask_word_begin > p.mask_word_end)
    return vsa::kBadArgument;
  p.dq = static_cast<__nv_bfloat16*>(dq);
  p.dk = static_cast<__nv_bfloat16*>(dk);
  p.dv = static_cast<__nv_bfloat16*>(dv);
  p.out_row_stride = out_row_stride;
  p.out_head_stride = out_head_stride;
  p.q_slot_row = q_slot_row;
  p.kv_slot_row = kv_slot_row;
  p.dq_pool = dq_pool;
  p.dk_pool = dk_pool;
  p.dv_pool = dv_pool;
  p.pool_f32 = pool_f32;
  p.q_block_coarse = q_block_coarse;
  p.kv_block_coarse = kv_block_coarse;
  p.q_sizes = q_sizes;
  p.dq_f32 = dq_f32;
  p.dk_f32 = dk_f32;
  p.dv_f32 = dv_f32;
  p.f32_accumulate = f32_accumulate;
  p.first_kv_blocks = (parts >> 8) & 0xFFFFF;
  if (p.first_kv_blocks > kv_blocks) p.first_kv_blocks = static_cast<int>(kv_blocks);
  p.q_out_rows = q_out_rows;
  p.kv_out_rows = kv_out_rows;
  p.q_slots = q_blocks * vsa::kBlock;
  p.kv_slots = kv_blocks * vsa::kBlock;
  p.q_blocks = static_cast<int>(q_blocks);
  p.kv_blocks = static_cast<int>(kv_blocks);
  p.heads = heads;
  p.scale = scale;
  p.status = status;
  cudaStream_t s = as_stream(stream);
  cudaError_t err = cudaSuccess;
  if (parts & 1)
    err = vsa::launch_build_kv_mask(indices, counts, index_head_stride, count_head_stride, capacity, heads,
                                    p.q_blocks, p.kv_blocks, kv_mask, p.mask_words, s);
  if (err == cudaSuccess && (parts & 2)) err = vsa::launch_fine_bwd_dq(p, s);
  if (err == cudaSuccess && (parts & 4)) err = vsa::launch_fine_bwd_dkv(p, s);
  return from_cuda(err);
}

}  // namespace

extern "C" {

int vsa_fine_bwd(const void* q, const void* k, const void* v, const void* d_o, int64_t q_blocks, int64_t kv_blocks,
                 int32_t heads, const int32_t* indices, const int32_t* counts, int64_t index_head_stride,
                 int64_t count_head_stride, int32_t capacity, const int32_t* q_sizes, const int32_t* kv_sizes,
                 float scale, const float* lse, const float* delta, uint32_t* kv_mask, void* dq, void* dk, void* dv,
                 int64_t q_out_rows, int64_t kv_out_rows, const int64_t* q_slot_row, const int64_t* kv_slot_row,
                 const void* dq_pool, const void* dk_pool, const void* dv_pool, int32_t pool_f32,
                 const int32_t* q_block_coarse, const int32_t* kv_block_coarse, float* dq_f32, float* dk_f32,
                 float* dv_f32, int32_t f32_accumulate, int32_t parts, int32_t* status, void* stream) {
  return fine_bwd_common(q, k, v, d_o, q_blocks, kv_blocks, heads, indices, counts, index_head_stride,
                         count_head_stride, capacity, q_sizes, kv_sizes, scale, lse, delta, kv_mask, dq, dk, dv,
                         static_cast<int64_t>(heads) * vsa::kDim, vsa::kDim, q_out_rows, kv_out_rows, q_slot_row,
                         kv_slot_row, dq_pool, dk_pool, dv_pool, pool_f32, q_block_coarse, kv_block_coarse, dq_f32,
                         dk_f32, dv_f32, f32_accumulate, parts, status, stream);
}

int vsa_fine_bwd_strided(const void* q, const void* k, const void* v, const void* d_o, int64_t q_blocks,
                         int64_t kv_blocks, int32_t heads, const int32_t* indices, const int32_t* counts,
                         int64_t index_head_stride, int64_t count_head_stride, int32_t capacity,
                         const int32_t* q_sizes, const int32_t* kv_sizes, float scale, const float* lse,
                         const float* delta, uint32_t* kv_mask, void* dq, void* dk, void* dv, int64_t out_row_stride,
                         int64_t out_head_stride, int64_t q_out_rows, int64_t kv_out_rows, const int64_t* q_slot_row,
                         const int64_t* kv_slot_row, const void* dq_pool, const void* dk_pool, const void* dv_pool,
                         int32_t pool_f32, const int32_t* q_block_coarse, const int32_t* kv_block_coarse,
                         int32_t parts, int32_t* status, void* stream) {
  return fine_bwd_common(q, k, v, d_o, q_blocks, kv_blocks, heads, indices, counts, index_head_stride,
                         count_head_stride, capacity, q_sizes, kv_sizes, scale, lse, delta, kv_mask, dq, dk, dv,
                         out_row_stride, out_head_stride, q_out_rows, kv_out_rows, q_slot_row, kv_slot_row, dq_pool,
                         dk_pool, dv_pool, pool_f32, q_block_coarse, kv_block_coarse, nullptr, nullptr, nullptr, 0,
                         parts, status, stream);
}

int vsa_fine_bwd_range(const void* q, const void* k, const void* v, const void* d_o, int64_t q_blocks,
                       int64_t kv_blocks, int32_t heads, const int32_t* indices, const int32_t* counts,
                       const int32_t* list_bounds, int64_t index_head_stride, int64_t count_head_stride,
                       int32_t bounds_stride, int32_t capacity, const int32_t* q_sizes, const int32_t* kv_sizes,
                       float scale, const float* lse, const float* delta, uint32_t* kv_mask, int32_t mask_word_begin,
                       int32_t mask_word_end, float* dq_f32, float* dk_f32, float* dv_f32, int32_t f32_accumulate,
                       int32_t parts, int32_t* status, void* stream) {
  if (mask_word_end < 0) return vsa::kBadArgument;
  return fine_bwd_common(q, k, v, d_o, q_blocks, kv_blocks, heads, indices, counts, index_head_stride,
                         count_head_stride, capacity, q_sizes, kv_sizes, scale, lse, delta, kv_mask, nullptr, nullptr,
                         nullptr, static_cast<int64_t>(heads) * vsa::kDim, vsa::kDim, 0, 0, nullptr, nullptr, nullptr,
                         nullptr, nullptr, 0, nullptr, nullptr, dq_f32, dk_f32, dv_f32, f32_accumulate, parts, status,
                         stream, list_bounds, bounds_stride, mask_word_begin, mask_word_end);
}

int vsa_list_bounds(const int32_t* lists, const int32_t* counts, int64_t rows, int32_t capacity, int32_t chunk_blocks,
                    int32_t chunks, int32_t* bounds, void* stream) {
  if (lists == nullptr || counts == nullptr || bounds == nullptr || rows < 0 || capacity <= 0 || chunk_blocks <= 0 ||
      chunks <= 0)
    return vsa::kBadArgument;
  return from_cuda(vsa::launch_list_bounds(lists, counts, rows, capacity, chunk_blocks, chunks, bounds,
                                           as_stream(stream)));
}

int vsa_partition_indices(const int32_t* index, const int32_t* counts, const int64_t* global_to_gather,
                          int32_t* out_lists, int32_t* out_counts, int64_t rows, int32_t capacity,
                          int32_t out_capacity, int32_t ring_size, int32_t peer_blocks, int64_t list_stride,
                          int64_t count_stride, void* stream) {
  if (index == nullptr || counts == nullptr || global_to_gather == nullptr || out_lists == nullptr ||
      out_counts == nullptr || rows < 0 || capacity <= 0 || out_capacity <= 0 || ring_size <= 0 || peer_blocks <= 0)
    return vsa::kBadArgument;
  return from_cuda(vsa::launch_partition_indices(index, counts, global_to_gather, out_lists, out_counts, rows,
                                                 capacity, out_capacity, ring_size, peer_blocks, list_stride,
                                                 count_stride, as_stream(stream)));
}

int vsa_merge_partial(float* out, float* lse, const void* part, const float* part_lse, int64_t slots, int32_t heads,
                      void* stream) {
  if (out == nullptr || lse == nullptr || part == nullptr || part_lse == nullptr || slots < 0 || heads <= 0)
    return vsa::kBadArgument;
  return from_cuda(vsa::launch_merge_partial(out, lse, static_cast<const __nv_bfloat16*>(part), part_lse, slots, heads,
                                             as_stream(stream)));
}

int vsa_gate_merge(const float* fine, const int64_t* slot_row, const int32_t* block_coarse, const void* gate,
                   const void* coarse, void* o_slots, void* out, int64_t blocks, int32_t heads, int64_t out_rows,
                   void* stream) {
  if (fine == nullptr || out == nullptr || blocks < 0 || heads <= 0) return vsa::kBadArgument;
  if (coarse != nullptr && (gate == nullptr || block_coarse == nullptr)) return vsa::kBadArgument;
  return from_cuda(vsa::launch_gate_merge(fine, slot_row, block_coarse, static_cast<const __nv_bfloat16*>(gate),
                                          static_cast<const __nv_bfloat16*>(coarse),
                                          static_cast<__nv_bfloat16*>(o_slots), static_cast<__nv_bfloat16*>(out),
                                          blocks, heads, out_rows, as_stream(stream)));
}

int vsa_grad_finish(const float* acc, const int64_t* slot_row, const void* pool, int32_t pool_f32,
                    const int32_t* block_map, const int32_t* block_sizes, void* out, int64_t blocks, int32_t heads,
                    int64_t out_rows, void* stream) {
  if (acc == nullptr || out == nullptr || blocks < 0 || heads <= 0) return vsa::kBadArgument;
  return from_cuda(vsa::launch_grad_finish(acc, slot_row, pool, pool_f32, block_map, block_sizes,
                                           static_cast<__nv_bfloat16*>(out), blocks, heads, out_rows,
                                           as_stream(stream)));
}

}  // extern "C"
