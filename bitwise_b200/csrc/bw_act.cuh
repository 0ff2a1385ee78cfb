// One source, two precisions: a file that includes this header is compiled once with
// -DBW_ACT_BF16=1 (activations, weights and caches in bfloat16) and once with -DBW_ACT_BF16=0
// (everything in float32). Arithmetic is float32 either way; only what is loaded and stored
// changes type. BW_FN gives the exported name of the precision.
#pragma once

#include "bw_common.cuh"

#ifndef BW_ACT_BF16
#error "compile with -DBW_ACT_BF16=0 or 1"
#endif

#if BW_ACT_BF16
typedef __nv_bfloat16 act_t;
#define BW_FN(name) bw_bf16_##name
#else
typedef float act_t;
#define BW_FN(name) bw_f32_##name
#endif

namespace bw {

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Sums over a warp and over a block of up to 1,024 threads in a fixed order: a butterfly inside
// the warp, then the warps' sums one after the other. Every thread gets the total.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* red /* 32 floats of shared memory */) {
  v = warp_sum(v);
  __syncthreads();  // red may still be read from the call before
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.0f;
  const int warps = (blockDim.x + 31) >> 5;
  for (int i = 0; i < warps; ++i) s = __fadd_rn(s, red[i]);
  return s;
}

}  // namespace bw
