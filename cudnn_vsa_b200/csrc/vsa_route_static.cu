// vsa_route_static: block routing for callers that are not allowed to allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc (or any allocator) around a routing call:
// an inference-runtime plugin whose `enqueue` hook must not allocate, a process whose device
// memory is entirely owned by another framework's pool, or code that runs where an allocation
// would serialise the device.  `vsa_route` needs a score matrix as scratch and asks the caller
// for it; this variant keeps that scratch inside the library instead, in a fixed 16 MiB array
// that lives in the module's device image.  Every GPU that loads the library holds those 16 MiB
// from load until exit, whether or not this entry point is ever called.
//
// Rules that follow from the shared array:
//   - One head's score matrix, (q_end - q_begin) * (kv_last - kv_first) floats, must fit in
//     16 MiB; larger regions are refused with VSA_STATUS_STATIC_SCRATCH (use vsa_route then).
//     More heads than fit are handled in several passes, as vsa_route does with a small scratch.
//   - The array keeps whatever the previous call left in it.  Nothing has to start at zero:
//     the score kernel writes every element the selection kernel reads, within the same call.
//   - All calls on a device share the one array, so two calls that overlap on the GPU (different
//     streams, or graphs replayed concurrently) race on it.  Keep them on one stream or order them.
//   - The first call on each device looks up the array's device address (a host-side query, no
//     allocation).  Make that first call before starting any stream capture.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/vsa_b200.h"
#include "vsa_common.cuh"
#include "vsa_kernels.h"

namespace {

constexpr long long kStaticScratchBytes = 16LL << 20;
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for the runtime; the address a kernel can use comes
// from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_route_scratch[kStaticScratchBytes];

std::mutex g_lock;
void* g_device_address[kMaxDevices] = {};

// Device address of the scratch array on the current device, or null with `*error` set.
float* scratch_for_current_device(int* error) {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
    *error = vsa::kCudaError;
    return nullptr;
  }
  std::lock_guard<std::mutex> guard(g_lock);
  if (g_device_address[device] == nullptr) {
    void* address = nullptr;
    if (cudaGetSymbolAddress(&address, g_route_scratch) != cudaSuccess || address == nullptr) {
      *error = vsa::kCudaError;
      return nullptr;
    }
    g_device_address[device] = address;
  }
  return static_cast<float*>(g_device_address[device]);
}

}  // namespace

extern "C" int vsa_route_static(const float* q_mean, const float* k_mean, int32_t heads, int32_t q_begin,
                                int32_t q_end, int32_t q_mean_offset, int32_t kv_first, int32_t kv_last,
                                int32_t k_mean_offset, int32_t keep, int32_t cursor, int32_t* indices,
                                int64_t index_head_stride, int32_t capacity, void* stream) {
  const int64_t rows = static_cast<int64_t>(q_end) - q_begin, region = static_cast<int64_t>(kv_last) - kv_first;
  if (q_mean == nullptr || k_mean == nullptr || indices == nullptr || heads <= 0 || rows < 0 || region <= 0 ||
      keep < 1 || keep > region || cursor < 0 || cursor + keep > capacity)
    return vsa::kBadArgument;
  if (rows == 0) return vsa::kOk;
  if (region * 4 > 200 * 1024) return vsa::kTooLarge;  // one score row must fit the selection kernel
  const int64_t per_head = rows * region * static_cast<int64_t>(sizeof(float));
  if (per_head > kStaticScratchBytes) return VSA_STATUS_STATIC_SCRATCH;
  int error = vsa::kOk;
  float* scratch = scratch_for_current_device(&error);
  if (scratch == nullptr) return error;
  int64_t chunk = kStaticScratchBytes / per_head;
  if (chunk > heads) chunk = heads;
  const vsa::RouteSpan span{q_begin, q_end, q_mean_offset, kv_first, kv_last, k_mean_offset, keep, cursor};
  for (int32_t head0 = 0; head0 < heads; head0 += static_cast<int32_t>(chunk)) {
    const int32_t now = heads - head0 < chunk ? heads - head0 : static_cast<int32_t>(chunk);
    if (vsa::launch_route_chunk(q_mean, k_mean, heads, head0, now, span, scratch, indices, index_head_stride,
                                capacity, static_cast<cudaStream_t>(stream)) != cudaSuccess)
      return vsa::kCudaError;
  }
  return vsa::kOk;
}
