// Shared helpers for the rdkv_b200 kernels (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "rdkv_b200.h"

namespace rdkv {

constexpr int D = RDKV_HEAD_DIM;
constexpr float INV_SQRT_D = 0.08838834764831845f;   // 1/sqrt(128)
constexpr int MAX_GROUP = 16;                        // query heads per KV head

// Per-thread record of the last failed launch, read back by rdkv_last_cuda_error().
extern thread_local int g_last_cuda_error;

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(e);
    return RDKV_ERR_LAUNCH;
  }
  return RDKV_OK;
}

__device__ __forceinline__ float load_q(const void* q, int dtype, int64_t idx) {
  if (dtype == RDKV_F16) return __half2float(reinterpret_cast<const __half*>(q)[idx]);
  if (dtype == RDKV_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(q)[idx]);
  return reinterpret_cast<const float*>(q)[idx];
}

__device__ __forceinline__ float h2f(uint16_t bits) {
  return __half2float(__ushort_as_half(bits));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Per-head row counts of a view, read from device memory at run time.
struct HeadCounts {
  int n2, n4, n8, n16, t_v;
};

__device__ __forceinline__ HeadCounts head_counts(const rdkv_layer_view& v, int h) {
  HeadCounts c;
  if (v.v_seg_bounds != nullptr) {
    c.n2 = v.v_seg_bounds[3 * h + 0];
    c.n4 = v.v_seg_bounds[3 * h + 1];
    c.n8 = v.v_seg_bounds[3 * h + 2];
  } else {
    c.n2 = v.n2; c.n4 = v.n4; c.n8 = v.n8;
  }
  c.n16 = (v.v16 == nullptr) ? 0 : (v.n_v16 != nullptr ? v.n_v16[h] : v.n_v16_shared);
  c.t_v = c.n2 + c.n4 + c.n8;
  return c;
}

}  // namespace rdkv
