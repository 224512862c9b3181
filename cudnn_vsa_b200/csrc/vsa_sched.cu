// Work counters of the persistent fine-attention kernels.
//
// A persistent launch hands out its tiles in order through one 32-bit counter in device memory
// (the first gridDim.x tiles are taken by block index, the rest by atomicAdd).  The counters live
// in a static device array, so a launch allocates nothing: the launcher takes the next of
// kCounterSlots slots round-robin and zeroes it with a 4-byte memset on the launch stream ahead
// of the kernel.  A slot comes round again after kCounterSlots further launches of this process
// on the device; launches that far apart are never in flight together (a stream or graph holds
// a handful of these kernels at a time).  The memset is an ordinary stream operation and is
// captured with the kernel when the launch is recorded into a CUDA graph; a captured launch keeps
// its slot for the life of the graph, so the one combination to avoid is replaying such a graph
// on one stream while another stream of the same device issues its thousandth launch since the
// capture at that very moment.
#include <atomic>
#include <mutex>

#include "vsa_kernels.h"

namespace vsa {

namespace {

constexpr int kCounterSlots = 1024;
constexpr int kMaxDevices = 64;

static __device__ unsigned g_tile_counters[kCounterSlots];

std::mutex g_lock;
unsigned* g_device_address[kMaxDevices] = {};
std::atomic<unsigned> g_next_slot{0};

}  // namespace

cudaError_t acquire_tile_counter(cudaStream_t stream, unsigned** counter) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  unsigned* base = nullptr;
  {
    std::lock_guard<std::mutex> guard(g_lock);
    if (g_device_address[device] == nullptr) {
      void* address = nullptr;
      if ((err = cudaGetSymbolAddress(&address, g_tile_counters)) != cudaSuccess) return err;
      g_device_address[device] = static_cast<unsigned*>(address);
    }
    base = g_device_address[device];
  }
  *counter = base + g_next_slot.fetch_add(1, std::memory_order_relaxed) % kCounterSlots;
  return cudaMemsetAsync(*counter, 0, sizeof(unsigned), stream);
}

}  // namespace vsa
