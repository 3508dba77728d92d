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

// Programmatic dependent launch: a kernel lets its successor start (be scheduled, run its prologue, prefetch
// constant data) as soon as all of its own CTAs have begun, and waits for its predecessor's completion and memory
// before it touches anything the predecessor wrote or may still read.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Optional timeline for tuning: when a trace buffer is set, thread 0 of block 0 of every kernel appends
// {kernel id, time it started, time its wait on the predecessor returned} (nanoseconds of %globaltimer).
// Each translation unit has its own copy of these two pointers; BSPEC_DEFINE_TRACE_SETTER exports its setter.
static __device__ unsigned long long* g_trace_buf = nullptr;   // [capacity][3]
static __device__ unsigned int* g_trace_cnt = nullptr;         // [2]: {next slot, capacity}

__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void trace_record(int kid, unsigned long long t_start) {
  if (g_trace_buf != nullptr && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
    const unsigned int slot = atomicAdd(g_trace_cnt, 1u);
    if (slot < g_trace_cnt[1]) {
      g_trace_buf[3 * slot] = (unsigned long long)kid;
      g_trace_buf[3 * slot + 1] = t_start;
      g_trace_buf[3 * slot + 2] = global_timer();
    }
  }
}
// a free-form mark from the calling thread of block 0 (phases inside a kernel)
__device__ __forceinline__ void trace_mark(int kid, unsigned long long t_from) {
  if (g_trace_buf != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
    const unsigned int slot = atomicAdd(g_trace_cnt, 1u);
    if (slot < g_trace_cnt[1]) {
      g_trace_buf[3 * slot] = (unsigned long long)kid;
      g_trace_buf[3 * slot + 1] = t_from;
      g_trace_buf[3 * slot + 2] = global_timer();
    }
  }
}
// Checked build (-DBSPEC_BOUNDS; set BSPEC_BOUNDS=1 in the environment when the library is built): indices that
// come from data (token ids, row numbers, block-table slots and the page ids in them) are compared with their
// ranges before they address memory with plain loads and stores.  The first one found outside is recorded as
// {code, value, limit, block} and the access is skipped: a wrong table then costs a wrong result and a report,
// not a fault.  Each translation unit has its own record; BSPEC_DEFINE_BOUNDS_REPORT exports its reader.
// Codes: 101 token id (embedding), 102 row (gather), 103 block-table slot and 104 page id (rotary + cache append),
// 105 / 106 the same in the q/k/v product's epilogue, 107 / 108 page id (attention over plain loads, float32 / bfloat16).  Copies through
// TMA need no such check: the tensor map clips them.
#ifdef BSPEC_BOUNDS
static __device__ int g_bounds[4] = {0, 0, 0, 0};
__device__ __forceinline__ bool in_range(long long v, long long n, int code) {
  if (v >= 0 && v < n) return true;
  if (atomicCAS(&g_bounds[0], 0, code) == 0) {
    g_bounds[1] = (int)max(-2147483647ll, min(2147483647ll, v));
    g_bounds[2] = (int)min(2147483647ll, n);
    g_bounds[3] = (int)blockIdx.x;
  }
  return false;
}
#else
__device__ __forceinline__ bool in_range(long long, long long, int) { return true; }
#endif
__device__ __forceinline__ void pdl_prologue(int kid = 0) {
  const unsigned long long t0 = g_trace_buf != nullptr ? global_timer() : 0ull;
  pdl_launch_dependents();
  pdl_wait();
  trace_record(kid, t0);
}

// Facts about a device are kept per device: a process may use several.
constexpr int kMaxDevices = 64;
inline int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev < 0 || dev >= kMaxDevices ? 0 : dev;
}
// Number of SMs of the current device (asked once per device).
inline int sm_count() {
  static int count[kMaxDevices] = {};
  const int dev = current_device();
  if (count[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    count[dev] = n > 0 ? n : 1;
  }
  return count[dev];
}

inline bool& pdl_enabled() {
  static bool on = true;
  return on;
}

// Launch with the programmatic-stream-serialization attribute (when enabled) and, optionally, a cluster along z.
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace bspec

#define BSPEC_LAUNCH(kernel, grid, block, smem, stream, ...) \
  (void)bspec::launch(kernel, dim3(grid), dim3(block), (size_t)(smem), stream, __VA_ARGS__)
#define BSPEC_LAUNCH_CHECK() (int)cudaGetLastError()
// Reads (and clears) the translation unit's record of the checked build into out4; returns 1 in a checked build,
// 0 otherwise (out4 zeroed), a negative CUDA error on failure.  Waits for the device.
#ifdef BSPEC_BOUNDS
#define BSPEC_DEFINE_BOUNDS_REPORT(name)                                                           \
  BSPEC_API int name(int* out4) {                                                                  \
    const int zero[4] = {0, 0, 0, 0};                                                              \
    cudaError_t e = cudaMemcpyFromSymbol(out4, bspec::g_bounds, sizeof(zero));                     \
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(bspec::g_bounds, zero, sizeof(zero));             \
    return e == cudaSuccess ? 1 : -(int)e;                                                         \
  }
#else
#define BSPEC_DEFINE_BOUNDS_REPORT(name)                                                           \
  BSPEC_API int name(int* out4) {                                                                  \
    out4[0] = out4[1] = out4[2] = out4[3] = 0;                                                     \
    return 0;                                                                                      \
  }
#endif
#define BSPEC_DEFINE_TRACE_SETTER(name)                                                            \
  BSPEC_API int name(unsigned long long* buf, unsigned int* cnt) {                                 \
    cudaError_t e = cudaMemcpyToSymbol(bspec::g_trace_buf, &buf, sizeof(buf));                     \
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(bspec::g_trace_cnt, &cnt, sizeof(cnt));           \
    return (int)e;                                                                                 \
  }
