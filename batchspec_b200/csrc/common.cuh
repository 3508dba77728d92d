// Shared helpers for the sm_100a kernels of batchspec_b200.
// Every exported entry point is `extern "C"`, takes raw device pointers plus
// explicit sizes and a stream, launches asynchronously and returns the launch's
// cudaError_t as an int (0 = ok).  Element types are passed as codes.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define BSPEC_F32 0
#define BSPEC_BF16 1

#define BSPEC_API extern "C" __attribute__((visibility("default")))

namespace bspec {

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// load element i of an array whose element type is given by a runtime code
__device__ __forceinline__ float load_as_f32(const void* p, int dtype, size_t i) {
  return dtype == BSPEC_F32 ? reinterpret_cast<const float*>(p)[i]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum with a fixed reduction tree (same order whatever else runs).
// `scratch` holds at least 32 floats of shared memory.  All threads get the sum.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

}  // namespace bspec

#define BSPEC_LAUNCH_CHECK() (int)cudaGetLastError()
