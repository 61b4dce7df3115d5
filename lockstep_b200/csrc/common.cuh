// Shared declarations of the CUDA sources: element types, the device error
// word, and small conversion helpers.  Every launcher is a plain C function
// (loaded with ctypes) that takes raw device pointers and the stream to launch
// on, allocates nothing, and returns 0 or a negative LS_E_* code for arguments
// it refuses, or the positive cudaError_t of a failed launch.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

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

// Launch constants that fix the order of a reduction are defined once, here or in the one
// source that uses them, and every source reports its own through ls_constants_<source>()
// as "name=value;..." so that a run can record the table it ran with.
#define LS_SPLIT 256         // keys of an attention split (fixed absolute positions)

struct LsConstant {
  const char* name;
  long long value;
};
static inline const char* ls_format_constants(char* buf, size_t size, const LsConstant* c, int count) {
  size_t at = 0;
  buf[0] = 0;
  for (int i = 0; i < count && at + 1 < size; ++i) {
    int n = snprintf(buf + at, size - at, "%s%s=%lld", i ? ";" : "", c[i].name, c[i].value);
    if (n < 0) break;
    at += (size_t)n;
  }
  return buf;
}

// Which kernels a process has launched (launcher calls, counted on the host): tests assert
// with it that the kernel they mean to check is the one that ran.
enum LsKernelId {
  LS_K_EMBED_GATHER = 0, LS_K_RMSNORM, LS_K_QK_NORM_ROPE, LS_K_QK_NORM_ROPE_WHOLE, LS_K_SILU_MUL,
  LS_K_GEMM_SIMT, LS_K_ATTENTION_TILE, LS_K_ATTENTION_DECODE, LS_K_ATTENTION_COMBINE, LS_K_ARGMAX,
  LS_K_SAMPLE, LS_K_GEMM_TC_FEW, LS_K_GEMM_TC_FEW_NORM, LS_K_GEMM_TC_FEW_QKV, LS_K_GEMM_TC_CLUSTER,
  LS_K_GEMM_TC_WALK, LS_K_GEMM_TC_ROWS, LS_K_GEMM_TC_ROWS_PAIR, LS_K_ATTENTION_DECODE_MMA,
  LS_K_ATTENTION_PREFILL_TC, LS_K_GEMM_SIMT_FEW, LS_K_GEMM_SIMT_MANY, LS_K_COUNT
};
#define LS_KERNEL_NAMES                                                                                  \
  "embed_gather,rmsnorm,qk_norm_rope_store,qk_norm_rope_store_whole,silu_mul,gemm_simt,attention_tile," \
  "attention_decode,attention_combine,argmax,sample,gemm_tc_few,gemm_tc_few_norm,gemm_tc_few_qkv,"      \
  "gemm_tc_cluster,gemm_tc_walk,gemm_tc_rows,gemm_tc_rows_pair,attention_decode_mma,attention_prefill_tc,"     \
  "gemm_simt_few,gemm_simt_many"
// one table per library: hidden, so that two libraries loaded into one process do not share it
__attribute__((visibility("hidden"))) inline unsigned long long ls_kernel_launches[LS_K_COUNT];
#define LS_COUNT(id) (++ls_kernel_launches[id])

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
