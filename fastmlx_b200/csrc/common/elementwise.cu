// Row gather (token embedding, and the choice of the rows whose logits are wanted),
// RMSNorm with the residual sum in front of it, and SiLU-and-multiply.
#include "common.cuh"

// out[t, :] = table[ids[t], :].  A bad id leaves a status code and a row of zeros.
template <typename T>
__global__ void gather_rows_kernel(const T* table, const int* ids, T* out,
                                   int d, long long nrows, int* status, int code) {
  pdl_wait();
  pdl_trigger();
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

// A table stored in 32-bit feeding bfloat16 activations: gather and round.
__global__ void gather_rows_f32_to_bf16_kernel(const float* table, const int* ids, bf16* out, int d, long long nrows,
                                               int* status, int code) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const long long id = ids[t];
  bf16* dst = out + (long long)t * d;
  const bool bad = id < 0 || id >= nrows;
  if (bad && threadIdx.x == 0) fmx_set_status(status, code, id, t);
  const float* src = table + (bad ? 0 : id) * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = __float2bfloat16_rn(bad ? 0.f : src[i]);
}

FMX_EXPORT int fmx_gather_rows_f32_to_bf16(const float* table, const int* ids, void* out, int n, int d,
                                           long long nrows, int* status, int code, cudaStream_t stream) {
  if (n == 0) return 0;
  if (n < 0 || d <= 0) return fmx_fail("fmx_gather_rows_f32_to_bf16: bad sizes n=%d d=%d", n, d);
  fmx_launch(gather_rows_f32_to_bf16_kernel, dim3(n), dim3(d >= 2048 ? 256 : 128), 0, stream, table, ids, (bf16*)out, d,
             nrows, status, code);
  FMX_LAUNCH_CHECK();
  return 0;
}

FMX_EXPORT int fmx_gather_rows(const void* table, const int* ids, void* out, int n, int d, long long nrows,
                               int dtype, int* status, int code, cudaStream_t stream) {
  if (n == 0) return 0;
  if (n < 0 || d <= 0) return fmx_fail("fmx_gather_rows: bad sizes n=%d d=%d", n, d);
  const int block = d >= 2048 ? 256 : 128;
  if (dtype == FMX_F32)
    gather_rows_kernel<float><<<n, block, 0, stream>>>((const float*)table, ids, (float*)out, d, nrows, status, code);
  else if (dtype == FMX_BF16)
    fmx_launch(gather_rows_kernel<bf16>, dim3(n), dim3(block), 0, stream, (const bf16*)table, ids, (bf16*)out, d, nrows,
               status, code);
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

// bfloat16 rows whose width is a multiple of 8: 16-byte loads, the row kept in registers
// between the sum of squares and the scaling (up to CH chunks of 8 per thread).  The sum of
// squares runs over a thread's elements in index order, then over the block in a fixed tree.
template <int BLOCK, int CH>
__global__ void __launch_bounds__(BLOCK)
add_rmsnorm_bf16_vec_kernel(const bf16* x, bf16* residual, const float* __restrict__ w, bf16* out, int d, float eps) {
  pdl_wait();
  pdl_trigger();
  const long long row = blockIdx.x;
  const int nvec = d / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * d);
  uint4* rr = residual ? reinterpret_cast<uint4*>(residual + row * d) : nullptr;
  float v[CH][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = threadIdx.x + c * BLOCK;
    if (i < nvec) {
      uint4 a = xr[i];
      const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
      if (rr) {
        uint4 b = rr[i];
        const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
        uint4 hsum;
        __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&hsum);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 fa = __bfloat1622float2(ap[e]), fb = __bfloat1622float2(bp[e]);
          hp[e] = __floats2bfloat162_rn(fa.x + fb.x, fa.y + fb.y);
          const float2 fh = __bfloat1622float2(hp[e]);
          v[c][2 * e] = fh.x;
          v[c][2 * e + 1] = fh.y;
        }
        rr[i] = hsum;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 fa = __bfloat1622float2(ap[e]);
          v[c][2 * e] = fa.x;
          v[c][2 * e + 1] = fa.y;
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss = fmaf(v[c][e], v[c][e], ss);
    }
  }
  ss = block_sum<BLOCK>(ss);
  const float rstd = 1.0f / sqrtf(ss / (float)d + eps);
  uint4* o = reinterpret_cast<uint4*>(out + row * d);
  const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = threadIdx.x + c * BLOCK;
    if (i < nvec) {
      const float4 w0 = w4[2 * i], w1 = w4[2 * i + 1];
      uint4 r;
      __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&r);
      rp[0] = __floats2bfloat162_rn(v[c][0] * rstd * w0.x, v[c][1] * rstd * w0.y);
      rp[1] = __floats2bfloat162_rn(v[c][2] * rstd * w0.z, v[c][3] * rstd * w0.w);
      rp[2] = __floats2bfloat162_rn(v[c][4] * rstd * w1.x, v[c][5] * rstd * w1.y);
      rp[3] = __floats2bfloat162_rn(v[c][6] * rstd * w1.z, v[c][7] * rstd * w1.w);
      o[i] = r;
    }
  }
}

static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

FMX_EXPORT int fmx_add_rmsnorm(const void* x, void* residual, const float* w, void* out, int rows, int d, float eps,
                               int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rows < 0 || d <= 0) return fmx_fail("fmx_add_rmsnorm: bad sizes rows=%d d=%d", rows, d);
  if (dtype == FMX_F32)
    add_rmsnorm_kernel<float, 256><<<rows, 256, 0, stream>>>((const float*)x, (float*)residual, w, (float*)out, d, eps);
  else if (dtype == FMX_BF16) {
    const bool vec = d % 8 == 0 && aligned16(x) && aligned16(out) && aligned16(w) && (!residual || aligned16(residual));
    if (vec && d <= 128 * 8)
      fmx_launch(add_rmsnorm_bf16_vec_kernel<128, 1>, dim3(rows), dim3(128), 0, stream, (const bf16*)x, (bf16*)residual, w,
                 (bf16*)out, d, eps);
    else if (vec && d <= 256 * 8)
      fmx_launch(add_rmsnorm_bf16_vec_kernel<256, 1>, dim3(rows), dim3(256), 0, stream, (const bf16*)x, (bf16*)residual, w,
                 (bf16*)out, d, eps);
    else if (vec && d <= 256 * 8 * 4)
      fmx_launch(add_rmsnorm_bf16_vec_kernel<256, 4>, dim3(rows), dim3(256), 0, stream, (const bf16*)x, (bf16*)residual, w,
                 (bf16*)out, d, eps);
    else
      add_rmsnorm_kernel<bf16, 256><<<rows, 256, 0, stream>>>((const bf16*)x, (bf16*)residual, w, (bf16*)out, d, eps);
  } else
    return fmx_fail("fmx_add_rmsnorm: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}

// out[t, i] = silu(gate_i) * up_i, silu(g) = g / (1 + exp(-g)), in 32-bit.  A row of gu holds
// 2 I values in blocks: `blk` gates, then their `blk` ups, and so on; blk = I is the plain
// layout [all gates | all ups].
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long long rows, int I, int blk) {
  const long long n = rows * I;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / I;
    const int i = (int)(idx - t * I);
    const int b = i / blk, j = i - b * blk;
    const float g = to_f(gu[t * 2 * I + (long long)b * 2 * blk + j]);
    const float u = to_f(gu[t * 2 * I + (long long)b * 2 * blk + blk + j]);
    out[idx] = from_f<T>(g / (1.0f + expf(-g)) * u);
  }
}

// bfloat16 with I a multiple of 8: eight elements per thread, 16-byte loads and stores.
__global__ void silu_mul_bf16_vec_kernel(const bf16* gu, bf16* out, int I, int blk) {
  pdl_wait();
  pdl_trigger();
  const long long t = blockIdx.y;
  const int nvec = I / 8, bvec = blk / 8;
  const uint4* gp = reinterpret_cast<const uint4*>(gu + t * 2 * I);
  uint4* op = reinterpret_cast<uint4*>(out + t * I);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += gridDim.x * blockDim.x) {
    const int b = i / bvec, j = i - b * bvec;
    const uint4 g4 = gp[b * 2 * bvec + j], u4 = gp[b * 2 * bvec + bvec + j];
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 r;
    __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
      r2[e] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
    }
    op[i] = r;
  }
}

FMX_EXPORT int fmx_silu_mul(const void* gu, void* out, int rows, int I, int blk, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rows < 0 || I <= 0) return fmx_fail("fmx_silu_mul: bad sizes rows=%d I=%d", rows, I);
  if (blk <= 0 || I % blk) return fmx_fail("fmx_silu_mul: %d is no multiple of the block size %d", I, blk);
  const long long n = (long long)rows * I;
  const int block = 256;
  const int grid = (int)((n + block - 1) / block < 148 * 16 ? (n + block - 1) / block : 148 * 16);
  if (dtype == FMX_F32)
    silu_mul_kernel<float><<<grid, block, 0, stream>>>((const float*)gu, (float*)out, rows, I, blk);
  else if (dtype == FMX_BF16) {
    if (I % 8 == 0 && blk % 8 == 0 && aligned16(gu) && aligned16(out) && rows <= 65535) {
      const int bx = (I / 8 + block - 1) / block;
      fmx_launch(silu_mul_bf16_vec_kernel, dim3(bx < 64 ? bx : 64, rows), dim3(block), 0, stream, (const bf16*)gu,
                 (bf16*)out, I, blk);
    } else {
      silu_mul_kernel<bf16><<<grid, block, 0, stream>>>((const bf16*)gu, (bf16*)out, rows, I, blk);
    }
  } else
    return fmx_fail("fmx_silu_mul: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}
