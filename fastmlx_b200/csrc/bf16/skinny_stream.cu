// out[M <= 16, N] = x . W^T for decode steps, one warp per 16-row tile of W, persistent.
//
// Same operand trick as skinny_gemm.cu (W rows are the A operand of mma.sync m16n8k16 and go
// from global memory straight into fragment registers, 16 contiguous bytes per thread, under a
// permutation of k shared with x), but a tile's whole K range (or one split of it) belongs to
// a single warp: no shared memory, no block-wide barrier, and the loads of the next four k
// blocks are in flight while the MMAs of the current four issue.  Blocks are persistent: each
// warp walks over (tile, split) work items, so there is no block launch and no reduction
// between tiles.  With K split over warps, partial tiles go to a workspace and the warp that
// draws the tile's last ticket adds them in split order.
//
// Epilogues: bias; residual (out = residual + product, in place when out is the residual);
// SiLU(gate) * up for a weight whose rows alternate in blocks of `blk` gate rows and their up
// rows (a warp then owns a gate tile and the matching up tile).
#include "common.cuh"

namespace {
constexpr int WARPS = 8;

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

template <int NT, int MT, typename TO>      // NT = 2: gate and up tiles; MT column tiles of 8 tokens
__global__ void __launch_bounds__(WARPS * 32, 2)
skinny_stream_kernel(const bf16* x, long long ldx, const bf16* __restrict__ W, long long ldw, TO* out, long long ldo,
                     int M, int N, int K, const float* __restrict__ bias, const bf16* residual, long long ldr, int blk,
                     int splits, float* ws, int* tickets) {
  constexpr int U = NT == 2 ? 2 : 4;         // k blocks per batch of loads: 64 registers of W per buffer pair
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int tiles = NT == 2 ? N / 32 : (N + 15) / 16;
  const int n_out = NT == 2 ? N / 2 : N;
  const int items = tiles * splits;
  const int nkb_all = (K + 31) / 32;
  const int per_split = (nkb_all + splits - 1) / splits;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  bool xok[MT];
  const bf16* xp[MT];
#pragma unroll
  for (int j = 0; j < MT; ++j) {
    xok[j] = 8 * j + g < M;
    xp[j] = x + (long long)(xok[j] ? 8 * j + g : 0) * ldx + 8 * t;
  }
  bool waited = false;

  for (int item = blockIdx.x * WARPS + warp; item < items; item += gridDim.x * WARPS) {
    const int tile = item / splits, split = item - tile * splits;
    int row0[NT], out0;
    if (NT == 2) {
      const int per = blk / 16;
      const int b = tile / per, j0 = (tile - b * per) * 16;
      row0[0] = b * 2 * blk + j0;
      row0[NT - 1] = row0[0] + blk;
      out0 = b * blk + j0;
    } else {
      row0[0] = tile * 16;
      out0 = row0[0];
    }
    const bf16* wp[NT][2];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      wp[i][0] = W + (long long)min(row0[i] + g, N - 1) * ldw + 8 * t;
      wp[i][1] = W + (long long)min(row0[i] + g + 8, N - 1) * ldw + 8 * t;
    }
    const int kb0 = split * per_split, kb1 = min(nkb_all, kb0 + per_split);
    float acc[NT][MT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
      for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

    uint4 a[2][U][NT][2];
    auto load_w = [&](int buf, int kb) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = (kb + u) * 32;
        const bool ok = kb + u < kb1 && k + 8 * t < K;
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          a[buf][u][i][0] = ok ? __ldcs(reinterpret_cast<const uint4*>(wp[i][0] + k)) : zero;
          a[buf][u][i][1] = ok ? __ldcs(reinterpret_cast<const uint4*>(wp[i][1] + k)) : zero;
        }
      }
    };
    auto compute = [&](int buf, int kb) {
      uint4 b[U][MT];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = (kb + u) * 32;
        const bool ok = kb + u < kb1 && k + 8 * t < K;
#pragma unroll
        for (int j = 0; j < MT; ++j) b[u][j] = (ok && xok[j]) ? __ldcg(reinterpret_cast<const uint4*>(xp[j] + k)) : zero;
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
          for (int j = 0; j < MT; ++j) {
            mma_bf16(acc[i][j], a[buf][u][i][0].x, a[buf][u][i][1].x, a[buf][u][i][0].y, a[buf][u][i][1].y, b[u][j].x, b[u][j].y);
            mma_bf16(acc[i][j], a[buf][u][i][0].z, a[buf][u][i][1].z, a[buf][u][i][0].w, a[buf][u][i][1].w, b[u][j].z, b[u][j].w);
          }
    };
    load_w(0, kb0);
    if (!waited) {                                    // W needs no predecessor; x does
      pdl_wait();
      waited = true;
    }
    for (int kb = kb0; kb < kb1; kb += 2 * U) {
      if (kb + U < kb1) load_w(1, kb + U);
      compute(0, kb);
      if (kb + U < kb1) {
        if (kb + 2 * U < kb1) load_w(0, kb + 2 * U);
        compute(1, kb + U);
      }
    }

    // this lane's results: rows g and g + 8 of the tile, tokens 8 j + 2 t and + 1
    auto finish = [&](int j, int e, float v0, float v1) {
      const int row = g + 8 * (e >> 1), tok = 8 * j + 2 * t + (e & 1);
      const int n = out0 + row;
      if (tok >= M || n >= n_out) return;
      float v = v0;
      if (NT == 2) {
        const float gate = bf16r(v0);
        v = gate / (1.0f + expf(-gate)) * bf16r(v1);
      }
      if (bias != nullptr) v += bias[n];
      if (residual != nullptr) v = bf16r(v) + __bfloat162float(residual[(long long)tok * ldr + n]);
      store_out<TO>(out + (long long)tok * ldo + n, v);
    };
    if (splits == 1) {
#pragma unroll
      for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) finish(j, e, acc[0][j][e], acc[NT - 1][j][e]);
      continue;
    }
    constexpr int PART = NT * MT * 128;                 // floats of one partial: 32 lanes x 4 per fragment
    float* mine = ws + ((long long)tile * splits + split) * PART;
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
      for (int j = 0; j < MT; ++j)
        __stcg(reinterpret_cast<float4*>(mine + (i * MT + j) * 128 + lane * 4),
               make_float4(acc[i][j][0], acc[i][j][1], acc[i][j][2], acc[i][j][3]));
    __threadfence();
    __syncwarp();
    int ticket = 0;
    if (lane == 0) ticket = atomicAdd(&tickets[tile], 1);
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    if (ticket != splits - 1) continue;
    __threadfence();
    const float* all = ws + (long long)tile * splits * PART;
    float tot[NT][MT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sp = 0; sp < splits; ++sp) {
          const float4 p = __ldcg(reinterpret_cast<const float4*>(all + (long long)sp * PART + (i * MT + j) * 128 + lane * 4));
          s.x += p.x; s.y += p.y; s.z += p.z; s.w += p.w;
        }
        tot[i][j][0] = s.x; tot[i][j][1] = s.y; tot[i][j][2] = s.z; tot[i][j][3] = s.w;
      }
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) finish(j, e, tot[0][j][e], tot[NT - 1][j][e]);
    if (lane == 0) tickets[tile] = 0;                   // ready for the next launch
  }
  if (!waited) pdl_wait();
}
}  // namespace

// Floats of workspace a call needs (0 for one split).
FMX_EXPORT long long fmx_skinny_stream_ws_floats(int M, int N, int splits, int blk) {
  if (splits <= 1) return 0;
  const long long tiles = blk > 0 ? N / 32 : (N + 15) / 16;
  return tiles * splits * (blk > 0 ? 2 : 1) * (M <= 8 ? 1 : 2) * 128;
}

// x [M <= 16, K] and W [N, K] bfloat16, rows 16-byte aligned.  bias float[n_out] or null;
// residual bfloat16 [M, n_out] (may be `out`) or null; blk > 0: W's rows alternate in blocks of
// blk gate rows and blk up rows and out is [M, N/2] = silu(gate) * up.  out bfloat16 (1) or
// float (0).  blocks: how many persistent blocks to launch (0: two per SM).
FMX_EXPORT int fmx_skinny_stream(const void* x, long long ldx, const void* W, long long ldw, void* out, long long ldo,
                                 int M, int N, int K, int out_dtype, const float* bias, const void* residual,
                                 long long ldr, int blk, int splits, float* ws, long long ws_floats, int* tickets,
                                 long long n_tickets, int blocks, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || M > 16 || N < 0 || K <= 0) return fmx_fail("fmx_skinny_stream: takes 1..16 rows, got M=%d N=%d K=%d", M, N, K);
  if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x & 15) || ((uintptr_t)W & 15))
    return fmx_fail("fmx_skinny_stream: rows must be 16-byte aligned (K=%d ldx=%lld ldw=%lld)", K, ldx, ldw);
  if (blk < 0 || (blk > 0 && (blk % 16 || N % (2 * blk))))
    return fmx_fail("fmx_skinny_stream: gate/up blocks of %d do not tile %d rows", blk, N);
  if (blk > 0 && M > 8) return fmx_fail("fmx_skinny_stream: the SiLU-mul epilogue takes at most 8 rows");
  if (splits < 1 || splits > 65535) return fmx_fail("fmx_skinny_stream: bad split count %d", splits);
  const int tiles = blk > 0 ? N / 32 : (N + 15) / 16;
  if (splits > 1 && (ws == nullptr || tickets == nullptr || ws_floats < fmx_skinny_stream_ws_floats(M, N, splits, blk) ||
                     n_tickets < tiles))
    return fmx_fail("fmx_skinny_stream: %d splits over %d tiles do not fit the workspace", splits, tiles);
  const long long items = (long long)tiles * splits;
  if (blocks <= 0) blocks = 2 * 148;
  const long long want = (items + WARPS - 1) / WARPS;
  const dim3 grid((unsigned)(want < blocks ? want : blocks)), block(WARPS * 32);
#define FMX_SS(NT_, MT_, TO_)                                                                                        \
  fmx_launch(skinny_stream_kernel<NT_, MT_, TO_>, grid, block, 0, stream, (const bf16*)x, ldx, (const bf16*)W, ldw,    \
             (TO_*)out, ldo, M, N, K, bias, (const bf16*)residual, ldr, blk, splits, ws, tickets)
  if (blk > 0) {
    if (out_dtype != FMX_BF16) return fmx_fail("fmx_skinny_stream: the SiLU-mul epilogue writes bfloat16");
    FMX_SS(2, 1, bf16);
  } else if (out_dtype == FMX_BF16) {
    if (M <= 8) FMX_SS(1, 1, bf16); else FMX_SS(1, 2, bf16);
  } else if (out_dtype == FMX_F32) {
    if (M <= 8) FMX_SS(1, 1, float); else FMX_SS(1, 2, float);
  } else {
    return fmx_fail("fmx_skinny_stream: unknown output dtype %d", out_dtype);
  }
#undef FMX_SS
  FMX_LAUNCH_CHECK();
  return 0;
}
