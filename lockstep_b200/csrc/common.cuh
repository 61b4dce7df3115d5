// Shared declarations of the CUDA sources: element types, the device error
// word, and small conversion helpers.  Every launcher is a plain C function
// (loaded with ctypes) that takes raw device pointers and the stream to launch
// on, allocates nothing, and returns 0 or a negative LS_E_* code for arguments
// it refuses, or the positive cudaError_t of a failed launch.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LS_API extern "C" __attribute__((visibility("default")))

// element types of tensors handed to a launcher
enum { LS_F32 = 0, LS_BF16 = 1 };

// refusals of a launcher (returned, nothing is launched)
enum {
  LS_E_DTYPE = -1,     // unsupported element type combination
  LS_E_SIZE = -2,      // a size the kernel does not take
  LS_E_ALIGN = -3,     // a pointer or stride that is not aligned as required
  LS_E_SMEM = -4,      // needs more shared memory than the device offers
};

// faults a kernel records in the device error word (first fault wins); the host
// reads the word after the step and raises.
enum {
  LS_DEV_OK = 0,
  LS_DEV_TOKEN_RANGE = 1,   // token id outside the embedding table
  LS_DEV_PAGE_RANGE = 2,    // block table names a page outside the pool
  LS_DEV_POSITION_RANGE = 3,// position outside the rotary table
  LS_DEV_WAIT_TIMEOUT = 4,  // a bounded wait on a barrier ran out
  LS_DEV_ROW_RANGE = 5,     // a row index outside its tensor
};

__device__ __forceinline__ void ls_record_fault(int* err, int code, int detail) {
  if (err != nullptr) {
    if (atomicCAS(err, 0, code) == 0) err[1] = detail;
  }
}

template <typename T>
__device__ __forceinline__ float ls_to_float(T v);
template <>
__device__ __forceinline__ float ls_to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float ls_to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

template <typename T>
__device__ __forceinline__ T ls_from_float(float v);
template <>
__device__ __forceinline__ float ls_from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 ls_from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float ls_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float ls_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a thread block in a fixed order: lanes by xor-tree, then warps
// ascending.  `scratch` holds one float per warp (at most 32).  All threads
// get the result.
__device__ __forceinline__ float ls_block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = ls_warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarps; ++w) total += scratch[w];
  return total;
}

// Programmatic dependent launch: a kernel may be scheduled while its predecessor
// in the stream still runs.  Every kernel calls ls_dependency_sync() before it
// touches global memory: it lets the next kernel start being scheduled, then
// waits until the previous kernel has completed and its writes are visible.
__device__ __forceinline__ void ls_dependency_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void ls_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void ls_dependency_sync() {
  ls_dependency_trigger();
  ls_dependency_wait();
}

// one switch per library (set through ls_set_dependent_launch_<library>)
inline int ls_dependent_launch = 1;

template <typename... KArgs, typename... Args>
static inline cudaError_t ls_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ls_dependent_launch ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

static inline int ls_launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}
