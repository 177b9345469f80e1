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

// One rotary pair, with the arithmetic pinned (no contraction left to the compiler) so that
// every kernel that rotates gets the same bits: (a, b) -> (a c - b s, b c + a s).
__device__ __forceinline__ void rope_pair(float a, float b, float s, float c, float& x, float& y) {
  x = __fmaf_rn(a, c, -__fmul_rn(b, s));
  y = __fmaf_rn(b, c, __fmul_rn(a, s));
}

// Programmatic dependent launch.  A kernel launched through fmx_launch may be scheduled
// while the kernel before it in the stream is still running: it does what needs no input
// from its predecessor (index arithmetic, reading weights), calls pdl_wait() before it reads
// or writes anything a predecessor may still touch, and only then calls pdl_trigger(), which
// lets the kernel after it be scheduled in turn.  pdl_wait() returns once every earlier
// kernel has finished and its writes are visible.  Triggering after the wait keeps the
// look-ahead one kernel deep: a kernel that triggers as its first statement lets the whole
// chain behind it become resident, where blocks of kernels far ahead sit on registers and
// shared memory that the running kernel needs (a decode step measured 10 % slower so).
// Without the launch attribute both calls are no-ops.  What a predecessor writes must not be
// read through the read-only data path (__ldg, or a const __restrict__ pointer, which lets
// the compiler choose that path): such loads count as invariant and may be moved above the
// wait.  Kernels launched this way therefore take their activations through plain pointers.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

bool fmx_pdl_enabled();
int fmx_num_sms();          // multiprocessors of the current device

template <typename... KArgs, typename... Args>
inline cudaError_t fmx_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = fmx_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with the blocks grouped into thread-block clusters of `cluster` blocks.
template <typename... KArgs, typename... Args>
inline cudaError_t fmx_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      dim3 cluster, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster.x;
  attr[0].val.clusterDim.y = cluster.y;
  attr[0].val.clusterDim.z = cluster.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = fmx_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Host side: the last error text of this thread, and the launch check every entry ends with.
const char* fmx_set_error(const char* msg);
int fmx_fail(const char* fmt, ...);
#define FMX_LAUNCH_CHECK()                                              \
  do {                                                                  \
    cudaError_t e_ = cudaGetLastError();                                \
    if (e_ != cudaSuccess) return fmx_fail("%s: %s", __func__, cudaGetErrorString(e_)); \
  } while (0)
