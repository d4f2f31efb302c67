// Shared helpers of the sequence-step kernels: storage types by dtype code, fp32 <-> storage conversion, block reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/omchat_b200_seq.h"
#include "omc_internal.h"

namespace omc {

typedef __nv_bfloat16 bf16_t;

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16_t* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16_t* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float seq_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float seq_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Sum over the block (<= 1024 threads); every thread gets the result. `red` is a __shared__ float[33].
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = seq_warp_sum(v);
  __syncthreads();  // red may still be read from a previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = seq_warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// Calls f(tag) with a null pointer of the storage type of dtype code `dt`; returns false for an unknown code.
#define OMC_DT_SWITCH(dt, T, ...)                 \
  if ((dt) == OMC_DT_F32) {                       \
    typedef float T;                              \
    __VA_ARGS__                                   \
  } else if ((dt) == OMC_DT_BF16) {               \
    typedef bf16_t T;                             \
    __VA_ARGS__                                   \
  } else {                                        \
    return set_error(OMC_ERR_ARG, "unknown dtype code"); \
  }

}  // namespace omc
