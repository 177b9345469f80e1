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

// residual' = round(residual + x) (32-bit sum, when residual is given; rounded to the residual's
// own type, which may be float beside bfloat16 activations: the stream then never rounds); out =
// residual' * 1/sqrt(mean(residual'^2) + eps) * w.  `init`: residual' = x (the stream's first
// value); x may be null when a residual is given (residual' = residual).  One block per row; the
// sum of squares is taken in a fixed order that depends on the row's width only.
template <typename T, typename TR, int BLOCK>
__global__ void add_rmsnorm_kernel(const T* x, TR* residual, const float* __restrict__ w, T* __restrict__ out, int d,
                                   float eps, int init) {
  pdl_wait();
  pdl_trigger();
  const long long row = blockIdx.x;
  const T* xr = x ? x + row * d : nullptr;
  TR* rr = residual ? residual + row * d : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += BLOCK) {
    float v = xr ? to_f(xr[i]) : 0.f;
    if (rr) {
      const TR h = from_f<TR>(init ? v : v + to_f(rr[i]));
      rr[i] = h;
      v = to_f(h);
    }
    ss = fmaf(v, v, ss);
  }
  ss = block_sum<BLOCK>(ss);
  const float rstd = 1.0f / sqrtf(ss / (float)d + eps);
  T* o = out + row * d;
  for (int i = threadIdx.x; i < d; i += BLOCK) o[i] = from_f<T>((rr ? to_f(rr[i]) : to_f(xr[i])) * rstd * w[i]);
}

// bfloat16 rows whose width is a multiple of 8: 16-byte loads, the row kept in registers
// between the sum of squares and the scaling (up to CH chunks of 8 per thread).  The sum of
// squares runs over a thread's elements in index order, then over the block in a fixed tree.
// RES_F32: the residual stream is float (two 16-byte accesses per eight elements).
template <int BLOCK, int CH, bool RES_F32>
__global__ void __launch_bounds__(BLOCK)
add_rmsnorm_bf16_vec_kernel(const bf16* x, void* residual, const float* __restrict__ w, bf16* out, int d, float eps,
                            int init) {
  pdl_wait();
  pdl_trigger();
  const long long row = blockIdx.x;
  const int nvec = d / 8;
  const uint4* xr = x ? reinterpret_cast<const uint4*>(x + row * d) : nullptr;
  uint4* rr = (residual && !RES_F32) ? reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(residual) + row * d) : nullptr;
  float4* rf = (residual && RES_F32) ? reinterpret_cast<float4*>(reinterpret_cast<float*>(residual) + row * d) : nullptr;
  float v[CH][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = threadIdx.x + c * BLOCK;
    if (i < nvec) {
      float xv[8];
      if (xr) {
        uint4 a = xr[i];
        const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 fa = __bfloat1622float2(ap[e]);
          xv[2 * e] = fa.x;
          xv[2 * e + 1] = fa.y;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) xv[e] = 0.f;
      }
      if (RES_F32 && rf) {
        float4 r0 = make_float4(0.f, 0.f, 0.f, 0.f), r1 = r0;
        if (!init) {
          r0 = rf[2 * i];
          r1 = rf[2 * i + 1];
        }
        v[c][0] = xv[0] + r0.x; v[c][1] = xv[1] + r0.y; v[c][2] = xv[2] + r0.z; v[c][3] = xv[3] + r0.w;
        v[c][4] = xv[4] + r1.x; v[c][5] = xv[5] + r1.y; v[c][6] = xv[6] + r1.z; v[c][7] = xv[7] + r1.w;
        rf[2 * i] = make_float4(v[c][0], v[c][1], v[c][2], v[c][3]);
        rf[2 * i + 1] = make_float4(v[c][4], v[c][5], v[c][6], v[c][7]);
      } else if (rr) {
        uint4 b = make_uint4(0u, 0u, 0u, 0u);
        if (!init) b = rr[i];
        const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
        uint4 hsum;
        __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&hsum);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 fb = __bfloat1622float2(bp[e]);
          hp[e] = __floats2bfloat162_rn(xv[2 * e] + fb.x, xv[2 * e + 1] + fb.y);
          const float2 fh = __bfloat1622float2(hp[e]);
          v[c][2 * e] = fh.x;
          v[c][2 * e + 1] = fh.y;
        }
        rr[i] = hsum;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[c][e] = xv[e];
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

template <bool RES_F32>
static void launch_add_rmsnorm_vec(const void* x, void* residual, const float* w, void* out, int rows, int d, float eps,
                                   int init, cudaStream_t stream) {
  if (d <= 128 * 8)
    fmx_launch(add_rmsnorm_bf16_vec_kernel<128, 1, RES_F32>, dim3(rows), dim3(128), 0, stream, (const bf16*)x, residual, w,
               (bf16*)out, d, eps, init);
  else if (d <= 256 * 8)
    fmx_launch(add_rmsnorm_bf16_vec_kernel<256, 1, RES_F32>, dim3(rows), dim3(256), 0, stream, (const bf16*)x, residual, w,
               (bf16*)out, d, eps, init);
  else
    fmx_launch(add_rmsnorm_bf16_vec_kernel<256, 4, RES_F32>, dim3(rows), dim3(256), 0, stream, (const bf16*)x, residual, w,
               (bf16*)out, d, eps, init);
}

// x, out: `dtype`; residual: `res_dtype` (float beside bfloat16 activations keeps the stream
// unrounded), or null.  init != 0: the residual is written, not read (the stream's first value).
// x may be null when there is a residual.
FMX_EXPORT int fmx_add_rmsnorm(const void* x, void* residual, const float* w, void* out, int rows, int d, float eps,
                               int dtype, int res_dtype, int init, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rows < 0 || d <= 0) return fmx_fail("fmx_add_rmsnorm: bad sizes rows=%d d=%d", rows, d);
  if (x == nullptr && (residual == nullptr || init)) return fmx_fail("fmx_add_rmsnorm: nothing to normalise");
  if (residual != nullptr && res_dtype != dtype && !(dtype == FMX_BF16 && res_dtype == FMX_F32))
    return fmx_fail("fmx_add_rmsnorm: a residual of type %d beside activations of type %d", res_dtype, dtype);
  const bool res_f32 = residual != nullptr && res_dtype == FMX_F32;
  if (dtype == FMX_F32)
    fmx_launch(add_rmsnorm_kernel<float, float, 256>, dim3(rows), dim3(256), 0, stream, (const float*)x, (float*)residual, w,
               (float*)out, d, eps, init);
  else if (dtype == FMX_BF16) {
    const bool vec = d % 8 == 0 && d <= 256 * 8 * 4 && aligned16(x) && aligned16(out) && aligned16(w) &&
                     (!residual || aligned16(residual));
    if (vec && res_f32)
      launch_add_rmsnorm_vec<true>(x, residual, w, out, rows, d, eps, init, stream);
    else if (vec)
      launch_add_rmsnorm_vec<false>(x, residual, w, out, rows, d, eps, init, stream);
    else if (res_f32)
      fmx_launch(add_rmsnorm_kernel<bf16, float, 256>, dim3(rows), dim3(256), 0, stream, (const bf16*)x, (float*)residual, w,
                 (bf16*)out, d, eps, init);
    else
      fmx_launch(add_rmsnorm_kernel<bf16, bf16, 256>, dim3(rows), dim3(256), 0, stream, (const bf16*)x, (bf16*)residual, w,
                 (bf16*)out, d, eps, init);
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
  const long long cap = (long long)fmx_num_sms() * 16;
  const int grid = (int)((n + block - 1) / block < cap ? (n + block - 1) / block : cap);
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

// out[r, :] = vec for every row: the bias laid under a library product that adds to what it finds
// (product and bias are then summed in 32-bit and rounded once).
template <typename T>
__global__ void fill_rows_kernel(const float* vec, T* out, long long rows, int cols, long long ldo) {
  pdl_wait();
  pdl_trigger();
  const long long n = rows * cols;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / cols;
    const int c = (int)(idx - r * cols);
    out[r * ldo + c] = from_f<T>(vec[c]);
  }
}

FMX_EXPORT int fmx_fill_rows(const float* vec, void* out, int rows, int cols, long long ldo, int dtype,
                             cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  if (rows < 0 || cols < 0 || ldo < cols) return fmx_fail("fmx_fill_rows: bad sizes rows=%d cols=%d ld=%lld", rows, cols, ldo);
  const long long n = (long long)rows * cols, cap = (long long)fmx_num_sms() * 16;
  const int block = 256;
  const int grid = (int)((n + block - 1) / block < cap ? (n + block - 1) / block : cap);
  if (dtype == FMX_F32)
    fmx_launch(fill_rows_kernel<float>, dim3(grid), dim3(block), 0, stream, vec, (float*)out, (long long)rows, cols, ldo);
  else if (dtype == FMX_BF16)
    fmx_launch(fill_rows_kernel<bf16>, dim3(grid), dim3(block), 0, stream, vec, (bf16*)out, (long long)rows, cols, ldo);
  else
    return fmx_fail("fmx_fill_rows: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}
