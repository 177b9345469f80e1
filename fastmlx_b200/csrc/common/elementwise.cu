// Row gather (token embedding, and the choice of the rows whose logits are wanted),
// RMSNorm with the residual sum in front of it, and SiLU-and-multiply.
#include "common.cuh"

// out[t, :] = table[ids[t], :].  A bad id leaves a status code and a row of zeros.
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ table, const int* __restrict__ ids, T* __restrict__ out,
                                   int d, long long nrows, int* status, int code) {
  const int t = blockIdx.x;
  const long long id = ids[t];
  T* dst = out + (long long)t * d;
  if (id < 0 || id >= nrows) {
    if (threadIdx.x == 0) fmx_set_status(status, code, id, t);
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = from_f<T>(0.f);
    return;
  }
  const T* src = table + id * d;
  const bool vec = ((size_t)d * sizeof(T)) % 16 == 0 && ((uintptr_t)src % 16 == 0) && ((uintptr_t)dst % 16 == 0);
  if (vec) {
    const int n = (int)((size_t)d * sizeof(T) / 16);
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int i = threadIdx.x; i < n; i += blockDim.x) d4[i] = s4[i];
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = src[i];
  }
}

FMX_EXPORT int fmx_gather_rows(const void* table, const int* ids, void* out, int n, int d, long long nrows,
                               int dtype, int* status, int code, cudaStream_t stream) {
  if (n == 0) return 0;
  if (n < 0 || d <= 0) return fmx_fail("fmx_gather_rows: bad sizes n=%d d=%d", n, d);
  const int block = d >= 2048 ? 256 : 128;
  if (dtype == FMX_F32)
    gather_rows_kernel<float><<<n, block, 0, stream>>>((const float*)table, ids, (float*)out, d, nrows, status, code);
  else if (dtype == FMX_BF16)
    gather_rows_kernel<bf16><<<n, block, 0, stream>>>((const bf16*)table, ids, (bf16*)out, d, nrows, status, code);
  else
    return fmx_fail("fmx_gather_rows: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}

// residual' = round(residual + x) (32-bit sum, when residual is given); out = residual' *
// 1/sqrt(mean(residual'^2) + eps) * w.  One block per row; the sum of squares is taken in
// a fixed order that depends on the row's width only.
template <typename T, int BLOCK>
__global__ void add_rmsnorm_kernel(const T* __restrict__ x, T* residual, const float* __restrict__ w,
                                   T* __restrict__ out, int d, float eps) {
  const long long row = blockIdx.x;
  const T* xr = x + row * d;
  T* rr = residual ? residual + row * d : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += BLOCK) {
    float v = to_f(xr[i]);
    if (rr) {
      const T h = from_f<T>(v + to_f(rr[i]));
      rr[i] = h;
      v = to_f(h);
    }
    ss = fmaf(v, v, ss);
  }
  ss = block_sum<BLOCK>(ss);
  const float rstd = 1.0f / sqrtf(ss / (float)d + eps);
  const T* src = rr ? rr : xr;
  T* o = out + row * d;
  for (int i = threadIdx.x; i < d; i += BLOCK) o[i] = from_f<T>(to_f(src[i]) * rstd * w[i]);
}

FMX_EXPORT int fmx_add_rmsnorm(const void* x, void* residual, const float* w, void* out, int rows, int d, float eps,
                               int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rows < 0 || d <= 0) return fmx_fail("fmx_add_rmsnorm: bad sizes rows=%d d=%d", rows, d);
  if (dtype == FMX_F32)
    add_rmsnorm_kernel<float, 256><<<rows, 256, 0, stream>>>((const float*)x, (float*)residual, w, (float*)out, d, eps);
  else if (dtype == FMX_BF16)
    add_rmsnorm_kernel<bf16, 256><<<rows, 256, 0, stream>>>((const bf16*)x, (bf16*)residual, w, (bf16*)out, d, eps);
  else
    return fmx_fail("fmx_add_rmsnorm: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}

// out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu(g) = g / (1 + exp(-g)), in 32-bit.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long long rows, int I) {
  const long long n = rows * I;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_f(gu[t * 2 * I + i]);
    const float u = to_f(gu[t * 2 * I + I + i]);
    out[idx] = from_f<T>(g / (1.0f + expf(-g)) * u);
  }
}

FMX_EXPORT int fmx_silu_mul(const void* gu, void* out, int rows, int I, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rows < 0 || I <= 0) return fmx_fail("fmx_silu_mul: bad sizes rows=%d I=%d", rows, I);
  const long long n = (long long)rows * I;
  const int block = 256;
  const int grid = (int)((n + block - 1) / block < 148 * 16 ? (n + block - 1) / block : 148 * 16);
  if (dtype == FMX_F32)
    silu_mul_kernel<float><<<grid, block, 0, stream>>>((const float*)gu, (float*)out, rows, I);
  else if (dtype == FMX_BF16)
    silu_mul_kernel<bf16><<<grid, block, 0, stream>>>((const bf16*)gu, (bf16*)out, rows, I);
  else
    return fmx_fail("fmx_silu_mul: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}
