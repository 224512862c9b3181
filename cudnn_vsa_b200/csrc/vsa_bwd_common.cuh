// Helpers shared by the two backward kernels of the fine attention.
#pragma once
#include "vsa_common.cuh"

namespace vsa {

constexpr float kLog2eBwd = 1.4426950408889634f;

VSA_DEVICE float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Pooled-mean gradient of `block` at column `col`, already divided by the block size.
VSA_DEVICE float pool_term(const void* pool, int pool_f32, const int32_t* block_coarse, int block, int size,
                           long long width, long long col) {
  long long prow = -1;
  if (pool != nullptr) prow = pool_f32 ? block : (block_coarse != nullptr ? block_coarse[block] : -1);
  if (prow < 0) return 0.f;
  const float inv = 1.f / static_cast<float>(size > 1 ? size : 1);
  const float value = pool_f32 ? static_cast<const float*>(pool)[prow * width + col]
                               : __bfloat162float(static_cast<const __nv_bfloat16*>(pool)[prow * width + col]);
  return value * inv;
}

}  // namespace vsa
