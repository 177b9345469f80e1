// A measuring kernel, not part of any step: how many clocks one tcgen05.mma of shape
// 128 x N x 16 takes when a single thread issues thousands of them back to back onto one
// accumulator, with A in shared or in tensor memory and B K-major or MN-major.  The
// operands are zeros; only the time is read.  It tells the tensor pipe's own rate apart from
// what a kernel's barriers and dependencies add (the attention kernels' P V products at head
// size 64 are N = 64: 48 clocks each where half of N = 128's 64 would be 32).
#include <cuda.h>
#include "common.cuh"
#include "tcgen05.cuh"

namespace {
using namespace fmx_tc;
constexpr int A_OFF = 0, B_OFF = 32 * 1024, OPERAND_BYTES = 96 * 1024, SMEM = OPERAND_BYTES + 1024;

// N_ > 0: shape and operand kinds are compile-time constants and nothing but the products
// themselves stands in the loop; N_ == 0: they are kernel arguments, and the thread computes
// descriptors and branches between the products, as a kernel's issuing thread does.
template <int N_, int TS_, int MN_>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int n_arg, int ts_arg, int mn_arg, int iters, long long* out) {
  const int n = N_ ? N_ : n_arg, a_in_tmem = N_ ? TS_ : ts_arg, b_mn_major = N_ ? MN_ : mn_arg;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  for (int i = threadIdx.x; i < OPERAND_BYTES / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = slot;
  if (threadIdx.x == 0) {
    const uint32_t idesc = make_idesc(128, n, b_mn_major);
    const uint32_t a = smem_u32(smem + A_OFF), b = smem_u32(smem + B_OFF);
    const long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        // MN-major B: 16 rows of the contraction per product, 64 columns per 128-byte row, the
        // next 64 columns 16 KB on; K-major B: 32 bytes further along each row
        const uint64_t bdesc = b_mn_major ? make_desc_mn128(b + k * 16 * 128, 16 * 1024) : make_desc_k128(b) + 2 * k;
        if (a_in_tmem) umma_f16_ts(tmem, tmem + 256 + 8 * k, bdesc, idesc, 1u);
        else umma_f16(tmem, make_desc_k128(a) + 2 * k, bdesc, idesc, 1u);
      }
    }
    const long long t1 = clock64();
    umma_commit(smem_u32(&bar));
    const bool ok = mbar_wait(smem_u32(&bar), 0);        // bounded
    out[0] = t1 - t0;
    out[1] = clock64() - t0;
    out[2] = ok ? 0 : 1;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

template <int N_, int TS_, int MN_>
int launch(int n, int ts, int mn, int iters, long long* out, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(mma_rate_kernel<N_, TS_, MN_>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) return fmx_fail("fmx_mma_rate: %d bytes of shared memory refused: %s", SMEM, cudaGetErrorString(e));
  mma_rate_kernel<N_, TS_, MN_><<<1, 128, SMEM, stream>>>(n, ts, mn, iters, out);
  FMX_LAUNCH_CHECK();
  return 0;
}
}  // namespace

// out[0]: clocks until the last of 4 * iters products was issued; out[1]: until all had
// completed; out[2]: 1 if the wait for completion ran out.  n in {64, 128, 256}; B MN-major
// only up to n = 128 (two 64-column blocks inside the zeroed operand area).
// `fixed` != 0: the kernel compiled for exactly this case (the pipe's own rate); 0: the one that
// takes the case as arguments.
FMX_EXPORT int fmx_mma_rate(int n, int a_in_tmem, int b_mn_major, int fixed, int iters, long long* out, cudaStream_t stream) {
  if ((n != 64 && n != 128 && n != 256) || iters <= 0 || iters > 100000 || (b_mn_major && n > 128))
    return fmx_fail("fmx_mma_rate: n=%d iters=%d mn_major=%d not measured", n, iters, b_mn_major);
  if (!fixed) return launch<0, 0, 0>(n, a_in_tmem, b_mn_major, iters, out, stream);
#define FMX_RATE_CASE(N_, TS_, MN_) \
  if (n == N_ && !a_in_tmem == !TS_ && !b_mn_major == !MN_) return launch<N_, TS_, MN_>(n, a_in_tmem, b_mn_major, iters, out, stream)
  FMX_RATE_CASE(64, 0, 0);
  FMX_RATE_CASE(128, 0, 0);
  FMX_RATE_CASE(256, 0, 0);
  FMX_RATE_CASE(64, 0, 1);
  FMX_RATE_CASE(128, 0, 1);
  FMX_RATE_CASE(64, 1, 1);
  FMX_RATE_CASE(128, 1, 1);
  FMX_RATE_CASE(128, 1, 0);
  FMX_RATE_CASE(256, 1, 0);
#undef FMX_RATE_CASE
  return fmx_fail("fmx_mma_rate: no kernel compiled for n=%d, A in tensor memory %d, B MN-major %d", n, a_in_tmem, b_mn_major);
}
