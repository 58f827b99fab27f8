// Shared device helpers for the sm_100a kernels: element conversion, warp and block
// reductions, vector access, and the error convention of the C entry points.
//
// Every entry point is `extern "C" int asb_<name>(..., cudaStream_t stream)`. It returns 0 on
// success; on a refused size or a failed launch it stores a message (asb_last_error) and
// returns non-zero. Nothing here allocates device memory: buffers come from the caller.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <utility>

namespace asb {

enum DType : int { kFloat32 = 0, kBFloat16 = 1 };

char* error_buffer();
int fail(const char* fmt, ...);
int check_launch(const char* what);

// Programmatic dependent launch. Every kernel of this library begins with pdl_wait(): when the
// launch carries the programmatic-serialization attribute, the grid may be scheduled while its
// predecessor in the stream is still running, and pdl_wait() is where it stops until that
// predecessor has completed and its writes are visible; what a kernel does before pdl_wait()
// (barrier set-up, tensor-memory allocation, loads of weights, which no kernel writes) overlaps the
// predecessor's tail. Without the attribute the instruction does nothing. pdl_enabled() is the
// library-wide switch (asb_set_pdl).
bool pdl_enabled();

// Every kernel of the library asks for the same split of an SM's memory between L1 and shared
// memory (the largest shared part, which the GEMM and attention kernels need). Blocks of a
// kernel with another split cannot join those still resident on an SM, which holds back the
// early start that a programmatic dependent launch gives: with one split for all, the decode-size
// GEMM calls measured 0.5 to 2 us shorter each. Set once per kernel function.
void prefer_shared_carveout(const void* kernel);

// Kernel launches made by this library so far (asb_launch_count reads it).
void count_launch();

template <typename... KArgs, typename... Args>
inline void launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                   Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = pdl_enabled() ? 1 : 0;
  prefer_shared_carveout((const void*)kernel);
  count_launch();
  cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);
}

// Among the rows of the requests that bring at most `limit` tokens, counted in request order,
// the flat row of number `index` (its request in *request); -1 if there are fewer such rows.
__device__ __forceinline__ int nth_short_row(const int* req_q_start, int R, int limit, int index, int* request) {
  int begin = req_q_start[0];
  for (int r = 0; r < R; ++r) {
    const int end = req_q_start[r + 1], n = end - begin;
    if (n <= limit) {
      if (index < n) { *request = r; return begin + index; }
      index -= n;
    }
    begin = end;
  }
  return -1;
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
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

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats of shared memory. Every
// thread gets the total. The order of the additions depends only on the block size.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float t = lane < nwarps ? scratch[lane] : 0.f;
  return warp_sum(t);
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float t = lane < nwarps ? scratch[lane] : -INFINITY;
  return warp_max(t);
}

}  // namespace asb

#define ASB_DISPATCH_DTYPE(dtype, T, ...)                         \
  do {                                                            \
    if ((dtype) == asb::kFloat32) {                               \
      using T = float;                                            \
      __VA_ARGS__;                                                \
    } else if ((dtype) == asb::kBFloat16) {                       \
      using T = __nv_bfloat16;                                    \
      __VA_ARGS__;                                                \
    } else {                                                      \
      return asb::fail("unknown dtype code %d", (int)(dtype));    \
    }                                                             \
  } while (0)
