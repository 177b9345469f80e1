// The skinny product of decode steps (at most 8 rows) with its neighbours folded in:
//   prologue : RMSNorm of the rows (x is then the residual stream; each block recomputes the
//              rows' 1/rms, one warp per row, and scales x on the fly as it builds fragments);
//   epilogue : residual add (out = residual + x W^T, in place when out is the residual), or
//              SiLU(gate) * up for a weight whose rows alternate in blocks of `blk` gate rows
//              and their `blk` up rows (a block then owns 16 gate rows and the 16 up rows
//              that go with them, and writes 16 columns of the activation).
// Rounding follows the unfused kernels: the normalised row, the product, gate and up are each
// rounded to bfloat16 where those kernels would have stored them.
//
// Operand layout, K interleaving over warps and the split-K ticket are those of
// skinny_gemm.cu; see there.
#include "common.cuh"

namespace {
constexpr int WARPS = 8;
constexpr int U = 4;

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ unsigned pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

template <int NT, typename TO>      // NT = 2: gate and up tiles of one block
__global__ void __launch_bounds__(WARPS * 32)
skinny_fused_kernel(const bf16* x, long long ldx, const bf16* __restrict__ W, long long ldw, TO* out, long long ldo,
                    int M, int N, int K, const float* __restrict__ norm_w, float eps, const bf16* residual,
                    long long ldr, int blk, float* ws, int* tickets) {
  __shared__ float red[WARPS][NT][16][9];
  __shared__ float rstd_s[8];
  __shared__ int last_ticket;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  int row0[NT], out0;
  if (NT == 2) {
    const int per = blk / 16;
    const int b = blockIdx.x / per, j0 = (blockIdx.x - b * per) * 16;
    row0[0] = b * 2 * blk + j0;
    row0[NT - 1] = row0[0] + blk;
    out0 = b * blk + j0;
  } else {
    row0[0] = blockIdx.x * 16;
    out0 = row0[0];
  }
  const int n_out = NT == 2 ? N / 2 : N;
  const bf16* wp[NT][2];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    wp[i][0] = W + (long long)min(row0[i] + g, N - 1) * ldw + 8 * t;
    wp[i][1] = W + (long long)min(row0[i] + g + 8, N - 1) * ldw + 8 * t;
  }
  const bool xok = g < M;
  const bf16* xp = x + (long long)(xok ? g : 0) * ldx + 8 * t;
  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;

  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  const int nkb_all = (K + 31) / 32;
  const int per_split = (nkb_all + gridDim.y - 1) / gridDim.y;
  const int kb0 = blockIdx.y * per_split;
  const int nkb = min(nkb_all, kb0 + per_split);

  uint4 a[U][NT][2];
  auto load_w = [&](int kb) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (kb + WARPS * u) * 32;
      const bool ok = kb + WARPS * u < nkb && k + 8 * t < K;
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        a[u][i][0] = ok ? __ldcs(reinterpret_cast<const uint4*>(wp[i][0] + k)) : zero;
        a[u][i][1] = ok ? __ldcs(reinterpret_cast<const uint4*>(wp[i][1] + k)) : zero;
      }
    }
  };
  int kb = kb0 + warp;
  if (kb < nkb) load_w(kb);                       // W is never written: ahead of the wait
  pdl_wait();
  pdl_trigger();

  float rstd = 1.f;
  if (norm_w != nullptr) {
    if (warp < M) {                               // one warp per row: 1 / rms over the whole of K
      const bf16* xr = x + (long long)warp * ldx;
      float ss = 0.f;
      for (int k = lane * 8; k < K; k += 32 * 8) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(xr + k));
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          ss = fmaf(f.x, f.x, ss);
          ss = fmaf(f.y, f.y, ss);
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) rstd_s[warp] = 1.0f / sqrtf(ss / (float)K + eps);
    }
    __syncthreads();
    rstd = xok ? rstd_s[g] : 0.f;
  }

  for (; kb < nkb; kb += WARPS * U) {
    uint4 b[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (kb + WARPS * u) * 32;
      const bool ok = kb + WARPS * u < nkb && k + 8 * t < K && xok;
      b[u] = ok ? __ldcg(reinterpret_cast<const uint4*>(xp + k)) : zero;
      if (norm_w != nullptr && ok) {
        const float4 w0 = __ldg(reinterpret_cast<const float4*>(norm_w + k + 8 * t));
        const float4 w1 = __ldg(reinterpret_cast<const float4*>(norm_w + k + 8 * t + 4));
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&b[u]);
        const float2 f0 = __bfloat1622float2(h[0]), f1 = __bfloat1622float2(h[1]), f2 = __bfloat1622float2(h[2]),
                     f3 = __bfloat1622float2(h[3]);
        uint4 r;
        r.x = pack2(f0.x * rstd * w0.x, f0.y * rstd * w0.y);
        r.y = pack2(f1.x * rstd * w0.z, f1.y * rstd * w0.w);
        r.z = pack2(f2.x * rstd * w1.x, f2.y * rstd * w1.y);
        r.w = pack2(f3.x * rstd * w1.z, f3.y * rstd * w1.w);
        b[u] = r;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        mma_bf16(acc[i], a[u][i][0].x, a[u][i][1].x, a[u][i][0].y, a[u][i][1].y, b[u].x, b[u].y);
        mma_bf16(acc[i], a[u][i][0].z, a[u][i][1].z, a[u][i][0].w, a[u][i][1].w, b[u].z, b[u].w);
      }
    if (kb + WARPS * U < nkb) load_w(kb + WARPS * U);
  }
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    red[warp][i][g][2 * t] = acc[i][0];
    red[warp][i][g][2 * t + 1] = acc[i][1];
    red[warp][i][g + 8][2 * t] = acc[i][2];
    red[warp][i][g + 8][2 * t + 1] = acc[i][3];
  }
  __syncthreads();

  constexpr int TILE = 16 * 8;
  const int splits = gridDim.y;
  auto finish = [&](int idx, float v0, float v1) {
    const int tok = idx / 16, row = idx - tok * 16;
    const int n = out0 + row;
    if (tok >= M || n >= n_out) return;
    float v = v0;
    if (NT == 2) {
      const float gte = bf16r(v0);
      v = gte / (1.0f + expf(-gte)) * bf16r(v1);
    }
    if (residual != nullptr) v = bf16r(v) + __bfloat162float(residual[(long long)tok * ldr + n]);
    store_out<TO>(out + (long long)tok * ldo + n, v);
  };
  if (splits == 1) {
    for (int idx = threadIdx.x; idx < TILE; idx += WARPS * 32) {
      const int tok = idx / 16, row = idx - tok * 16;
      float v[NT];
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        v[i] = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v[i] += red[w][i][row][tok];
      }
      finish(idx, v[0], v[NT - 1]);
    }
    return;
  }
  float* mine = ws + ((long long)blockIdx.x * splits + blockIdx.y) * (NT * TILE);
  for (int idx = threadIdx.x; idx < NT * TILE; idx += WARPS * 32) {
    const int i = idx / TILE, e = idx - i * TILE;
    const int tok = e / 16, row = e - tok * 16;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) v += red[w][i][row][tok];
    __stcg(mine + idx, v);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last_ticket = atomicAdd(&tickets[blockIdx.x], 1);
  __syncthreads();
  if (last_ticket != splits - 1) return;
  __threadfence();
  const float* all = ws + (long long)blockIdx.x * splits * (NT * TILE);
  for (int idx = threadIdx.x; idx < TILE; idx += WARPS * 32) {
    float v[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      v[i] = 0.f;
      for (int sp = 0; sp < splits; ++sp) v[i] += __ldcg(all + (long long)sp * (NT * TILE) + i * TILE + idx);
    }
    finish(idx, v[0], v[NT - 1]);
  }
  if (threadIdx.x == 0) tickets[blockIdx.x] = 0;
}
}  // namespace

FMX_EXPORT long long fmx_skinny_fused_ws_floats(int N, int splits, int dual) {
  return splits <= 1 ? 0 : (long long)((N + 15) / 16) * splits * 128;      // dual: N/32 blocks of two tiles
}

// x [M <= 8, K] and W [N, K] bfloat16, rows 16-byte aligned.  norm_w (float[K]) or null; residual
// (bfloat16 [M, n_out], may be `out` itself) or null; blk > 0: W's rows alternate in blocks of
// blk gate rows and blk up rows, out is [M, N/2] = silu(gate) * up.  out bfloat16 (1) or float (0).
FMX_EXPORT int fmx_skinny_fused(const void* x, long long ldx, const void* W, long long ldw, void* out, long long ldo,
                                int M, int N, int K, int out_dtype, const float* norm_w, float eps,
                                const void* residual, long long ldr, int blk, int splits, float* ws,
                                long long ws_floats, int* tickets, long long n_tickets, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || M > 8 || N < 0 || K <= 0) return fmx_fail("fmx_skinny_fused: takes 1..8 rows, got M=%d N=%d K=%d", M, N, K);
  if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x & 15) || ((uintptr_t)W & 15) || (norm_w && ((uintptr_t)norm_w & 15)))
    return fmx_fail("fmx_skinny_fused: rows must be 16-byte aligned (K=%d ldx=%lld ldw=%lld)", K, ldx, ldw);
  if (blk < 0 || (blk > 0 && (blk % 16 || N % (2 * blk))))
    return fmx_fail("fmx_skinny_fused: gate/up blocks of %d do not tile %d rows", blk, N);
  if (splits < 1 || splits > 65535) return fmx_fail("fmx_skinny_fused: bad split count %d", splits);
  const int tiles = blk > 0 ? N / 32 : (N + 15) / 16;
  if (splits > 1 && (ws == nullptr || tickets == nullptr || ws_floats < (long long)tiles * splits * (blk > 0 ? 256 : 128) ||
                     n_tickets < tiles))
    return fmx_fail("fmx_skinny_fused: %d splits over %d tiles do not fit the workspace", splits, tiles);
  const dim3 grid(tiles, splits), block(WARPS * 32);
#define FMX_SF(NT_, TO_)                                                                                          \
  fmx_launch(skinny_fused_kernel<NT_, TO_>, grid, block, 0, stream, (const bf16*)x, ldx, (const bf16*)W, ldw,      \
             (TO_*)out, ldo, M, N, K, norm_w, eps, (const bf16*)residual, ldr, blk, ws, tickets)
  if (blk > 0) {
    if (out_dtype != FMX_BF16) return fmx_fail("fmx_skinny_fused: the SiLU-mul epilogue writes bfloat16");
    FMX_SF(2, bf16);
  } else if (out_dtype == FMX_BF16) {
    FMX_SF(1, bf16);
  } else if (out_dtype == FMX_F32) {
    FMX_SF(1, float);
  } else {
    return fmx_fail("fmx_skinny_fused: unknown output dtype %d", out_dtype);
  }
#undef FMX_SF
  FMX_LAUNCH_CHECK();
  return 0;
}
