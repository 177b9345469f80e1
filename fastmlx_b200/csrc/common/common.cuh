// Shared helpers of the kernels: element types, conversions, the status word, launch checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define FMX_EXPORT extern "C" __attribute__((visibility("default")))

enum FmxDtype { FMX_F32 = 0, FMX_BF16 = 1 };

// Codes a kernel leaves in status[0] instead of trapping (status[1] = the bad value,
// status[2] = where).  The first code wins.
enum FmxStatus { FMX_OK = 0, FMX_BAD_TOKEN = 1, FMX_BAD_SLOT = 2, FMX_BAD_PAGE = 3, FMX_BAD_ROW = 4, FMX_WAIT_EXPIRED = 5 };

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ void fmx_set_status(int* status, int code, long long value, int where) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) {
    status[1] = (int)value;
    status[2] = where;
  }
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

// Sum over a block of BLOCK threads in a fixed order; every thread gets the result.
template <int BLOCK> __device__ __forceinline__ float block_sum(float v) {
  __shared__ float part[BLOCK / 32];
  __shared__ float total;
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float s = threadIdx.x < BLOCK / 32 ? part[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) total = s;
  }
  __syncthreads();
  float r = total;
  __syncthreads();
  return r;
}

// Host side: the last error text of this thread, and the launch check every entry ends with.
const char* fmx_set_error(const char* msg);
int fmx_fail(const char* fmt, ...);
#define FMX_LAUNCH_CHECK()                                              \
  do {                                                                  \
    cudaError_t e_ = cudaGetLastError();                                \
    if (e_ != cudaSuccess) return fmx_fail("%s: %s", __func__, cudaGetErrorString(e_)); \
  } while (0)
