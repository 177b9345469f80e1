// out[M, N] = x[M, K] . W[N, K]^T for at most 16 rows, one block per 8 (or 16) output features
// and the whole of K: no sum is split over blocks, so there is no workspace, no ticket and no
// second pass, and the order of the sum is fixed by construction.
//
// The rows of x are the A operand of mma.sync m16n8k16 (padded to 16), eight rows of W the B
// operand.  As in skinny_gemm.cu nothing is staged in shared memory: the sum over k does not
// care in which order k is visited, so each thread loads 16 contiguous bytes of a W row and
// of an x row straight into registers and hands them to two MMAs under a permutation of k
// that is the same for both operands.  The 8 or 16 warps of a block take interleaved 32-wide
// slices of K and add their partial tiles through shared memory in warp order.
//
// With 8 features per block a 2048-wide output still makes 256 blocks, enough to keep every
// SM streaming, where 16-row tiles had to split K over blocks and reduce through L2.
//
// Epilogues: bias; residual add (in place when out is the residual); SiLU(gate) * up for a
// weight whose rows alternate in blocks of `blk` gate rows and their `blk` up rows.
#include "common.cuh"

namespace {

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

// NT tiles of 8 features per block; HI: rows 8..15 of x exist; DUAL: the NT tiles are gate
// tiles and each has an up tile `blk` rows further on.
// What the greedy head leaves instead of logits: per row the best (value, index) as one 64-bit word that
// atomicMax orders (the value's bits made monotonic above, the index inverted below, so that the lower
// index wins a tie), a ticket that tells the last block, and the chosen ids.
struct GreedyOut {
  unsigned long long* best;      // [16], zero between launches
  int* ticket;                   // [1], zero between launches
  int* ids;                      // [M]
  int blocks;                    // feature blocks of the product; the grid may be smaller and then walks them
};
__device__ __forceinline__ unsigned long long greedy_key(float v, int n) {
  unsigned u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);                  // monotonic in v; every real key is above 0
  return ((unsigned long long)u << 32) | (unsigned)(0x7fffffff - n);
}

template <int NT, bool HI, bool DUAL, int U, int WARPS, typename TO, bool GREEDY = false>
__global__ void __launch_bounds__(WARPS * 32)
gemv_kernel(const bf16* x, long long ldx, const bf16* __restrict__ W, long long ldw, const float* __restrict__ bias,
            const bf16* residual, long long ldr, TO* out, long long ldo, int M, int N, int K, int blk,
            GreedyOut greedy = GreedyOut{nullptr, nullptr, nullptr, 0}) {
  constexpr int TILES = DUAL ? 2 * NT : NT;
  constexpr int ROWS = HI ? 16 : 8;
  __shared__ float red[WARPS][TILES][ROWS][9];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  // The greedy head walks its feature blocks with a grid that is resident at once (a vocabulary of 128,256 makes
  // 4,008 blocks): a block asks for the first W tiles of its next feature block before it reduces the one it has
  // just summed, so the reduction and the next block's first loads overlap.  Every other product: one feature
  // block per thread block.
  constexpr bool WALK = GREEDY;
  int vb = blockIdx.x;
  const int n_vb = WALK ? greedy.blocks : (int)gridDim.x;
  // the first W row of each tile, and the first output column of the block
  int row0[TILES], out0;
  if (DUAL) {
    const int per = blk / (8 * NT);
    const int b = blockIdx.x / per, j0 = (blockIdx.x - b * per) * 8 * NT;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      row0[i] = b * 2 * blk + j0 + 8 * i;
      row0[NT + i] = row0[i] + blk;
    }
    out0 = b * blk + j0;
  } else {
#pragma unroll
    for (int i = 0; i < TILES; ++i) row0[i] = vb * 8 * NT + 8 * i;
    out0 = row0[0];
  }
  const int n_out = DUAL ? N / 2 : N;
  const bf16* wp[TILES];
#pragma unroll
  for (int i = 0; i < TILES; ++i) wp[i] = W + (long long)min(row0[i] + g, N - 1) * ldw + 8 * t;
  const bool ok_lo = g < M, ok_hi = HI && g + 8 < M;
  const bf16* xlo = x + (long long)(ok_lo ? g : 0) * ldx + 8 * t;
  const bf16* xhi = x + (long long)(ok_hi ? g + 8 : 0) * ldx + 8 * t;
  float acc[TILES][4];
#pragma unroll
  for (int i = 0; i < TILES; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;

  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  const int nkb = (K + 31) / 32;
  uint4 b[U][TILES];
  auto load_w = [&](int kb) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (kb + WARPS * u) * 32;
      const bool ok = kb + WARPS * u < nkb && k + 8 * t < K;     // K is a multiple of 8: all 16 bytes or none
#pragma unroll
      for (int i = 0; i < TILES; ++i) b[u][i] = ok ? __ldcs(reinterpret_cast<const uint4*>(wp[i] + k)) : zero;
    }
  };
  int kb = warp;
  if (kb < nkb) load_w(kb);                       // W is never written by a kernel: ahead of the wait
  pdl_wait();                                     // x is; it is read through plain loads, after the wait
  __shared__ int drew_last;
  while (true) {
  for (; kb < nkb; kb += WARPS * U) {
    uint4 alo[U], ahi[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (kb + WARPS * u) * 32;
      const bool ok = kb + WARPS * u < nkb && k + 8 * t < K;
      alo[u] = (ok && ok_lo) ? __ldcg(reinterpret_cast<const uint4*>(xlo + k)) : zero;
      ahi[u] = (HI && ok && ok_hi) ? __ldcg(reinterpret_cast<const uint4*>(xhi + k)) : zero;
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int i = 0; i < TILES; ++i) {
        mma_bf16(acc[i], alo[u].x, ahi[u].x, alo[u].y, ahi[u].y, b[u][i].x, b[u][i].y);
        mma_bf16(acc[i], alo[u].z, ahi[u].z, alo[u].w, ahi[u].w, b[u][i].z, b[u][i].w);
      }
    if (kb + WARPS * U < nkb) load_w(kb + WARPS * U);
  }
  const int out_now = out0;
  const bool more = WALK && vb + (int)gridDim.x < n_vb;
  if (more) {                                     // the next feature block's first tiles, under the reduction below
    vb += gridDim.x;
    out0 = vb * 8 * NT;
#pragma unroll
    for (int i = 0; i < TILES; ++i) wp[i] = W + (long long)min(out0 + 8 * i + g, N - 1) * ldw + 8 * t;
    kb = warp;
    if (kb < nkb) load_w(kb);
  } else {
    pdl_trigger();                                // the block's loads are done: room for the next kernel's
  }
#pragma unroll
  for (int i = 0; i < TILES; ++i) {
    red[warp][i][g][2 * t] = acc[i][0];
    red[warp][i][g][2 * t + 1] = acc[i][1];
    if (HI) {
      red[warp][i][g + 8][2 * t] = acc[i][2];
      red[warp][i][g + 8][2 * t + 1] = acc[i][3];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < NT * ROWS * 8; idx += WARPS * 32) {
    const int f = idx & 7, rest = idx >> 3, i = rest % NT, tok = rest / NT;      // consecutive threads: consecutive features
    const int n = out_now + 8 * i + f;
    if (GREEDY) {
      // the row's 8 * NT logits of this block sit in consecutive lanes of whole warps: their best by a
      // shuffle tree, then one atomicMax per row and block
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) v += red[w][i][tok][f];
      unsigned long long key = (tok < M && n < n_out) ? greedy_key(v, n) : 0ull;
#pragma unroll
      for (int o = 4 * NT; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
        key = other > key ? other : key;
      }
      if ((idx & (8 * NT - 1)) == 0 && tok < M && key != 0ull) atomicMax(&greedy.best[tok], key);
      continue;
    }
    if (tok >= M || n >= n_out) continue;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) v += red[w][i][tok][f];
    if (DUAL) {
      float up = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) up += red[w][NT + i][tok][f];
      const float gte = bf16r(v);
      v = gte / (1.0f + expf(-gte)) * bf16r(up);
    }
    if (bias != nullptr) v += bias[n];
    if (residual != nullptr) v = bf16r(v) + __bfloat162float(residual[(long long)tok * ldr + n]);
    store_out<TO>(out + (long long)tok * ldo + n, v);
  }
  if (!more) break;
  __syncthreads();                                // the sums in `red` are read; the next feature block may write them
#pragma unroll
  for (int i = 0; i < TILES; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
  }
  if (GREEDY) {
    // The block that draws the last ticket turns the rows' best words into ids and leaves the words and
    // the ticket at zero for the next launch.  Nobody waits for anybody.
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      drew_last = atomicAdd(greedy.ticket, 1) == (int)gridDim.x - 1;
      if (drew_last) __threadfence();
    }
    __syncthreads();
    if (!drew_last) return;
    if (threadIdx.x < M) {
      const unsigned long long key = atomicExch(&greedy.best[threadIdx.x], 0ull);
      greedy.ids[threadIdx.x] = key == 0ull ? 0 : 0x7fffffff - (int)(unsigned)(key & 0xffffffffull);
    }
    if (threadIdx.x == 0) *greedy.ticket = 0;
  }
}

template <int NT, bool HI, bool DUAL, int U, int WARPS, typename TO>
void launch(const void* x, long long ldx, const void* W, long long ldw, const float* bias, const void* residual,
            long long ldr, void* out, long long ldo, int M, int N, int K, int blk, cudaStream_t stream) {
  const int n_out = DUAL ? N / 2 : N;
  fmx_launch(gemv_kernel<NT, HI, DUAL, U, WARPS, TO>, dim3((n_out + 8 * NT - 1) / (8 * NT)), dim3(WARPS * 32), 0, stream,
             (const bf16*)x, ldx, (const bf16*)W, ldw, bias, (const bf16*)residual, ldr, (TO*)out, ldo, M, N, K, blk,
             GreedyOut{nullptr, nullptr, nullptr, 0});
}
}  // namespace

// The output head of a decode step with the greedy choice made in the same pass: ids[m] = the index of the
// largest of x[m] . W[n]^T over n (the lowest index on ties), for at most 16 rows; no logits are written.
// best: 16 64-bit words, ticket: one int, both zero before the first call (every call leaves them zero).
// Calls that share them must not overlap on the GPU.
FMX_EXPORT int fmx_gemv_argmax(const void* x, long long ldx, const void* W, long long ldw, int* ids, void* best, int* ticket,
                               int M, int N, int K, cudaStream_t stream) {
  if (M == 0) return 0;
  if (M < 0 || M > 16 || N <= 0 || N > 0x7fffffff - 1 || K <= 0) return fmx_fail("fmx_gemv_argmax: takes 1..16 rows, got M=%d N=%d K=%d", M, N, K);
  if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x & 15) || ((uintptr_t)W & 15))
    return fmx_fail("fmx_gemv_argmax: rows must be 16-byte aligned (K=%d ldx=%lld ldw=%lld)", K, ldx, ldw);
  if (ids == nullptr || best == nullptr || ticket == nullptr || ((uintptr_t)best & 7)) return fmx_fail("fmx_gemv_argmax: needs ids, best words and a ticket");
  const int blocks = (N + 31) / 32;
  const GreedyOut g{(unsigned long long*)best, ticket, ids, blocks};
  const int resident = 2 * fmx_num_sms();          // two blocks of 256 threads and about 124 registers fit an SM
  const dim3 grid(blocks < resident ? blocks : resident);
  if (M > 8)
    fmx_launch(gemv_kernel<4, true, false, 2, 8, float, true>, grid, dim3(256), 0, stream, (const bf16*)x, ldx, (const bf16*)W, ldw,
               (const float*)nullptr, (const bf16*)nullptr, 0LL, (float*)nullptr, 0LL, M, N, K, 0, g);
  else
    fmx_launch(gemv_kernel<4, false, false, 4, 8, float, true>, grid, dim3(256), 0, stream, (const bf16*)x, ldx, (const bf16*)W, ldw,
               (const float*)nullptr, (const bf16*)nullptr, 0LL, (float*)nullptr, 0LL, M, N, K, 0, g);
  FMX_LAUNCH_CHECK();
  return 0;
}

// Output features per block when the caller leaves the choice open: 32 once that still gives
// every SM a block, else 16 (wider blocks re-read x less and keep more of W in flight per block,
// but too few of them leave SMs idle); halved until it tiles the gate/up blocks.
FMX_EXPORT int fmx_gemv_plan_width(int n_out, int blk, int sms) {
  if (sms <= 0) sms = fmx_num_sms();
  int wide = n_out / 32 >= sms ? 32 : 16;
  while (blk > 0 && blk % wide) wide /= 2;
  return wide;
}
// Warps per block: fewer blocks than SMs over a long K keep enough bytes in flight only with 16.
FMX_EXPORT int fmx_gemv_plan_warps(int n_out, int K, int wide, int sms) {
  if (sms <= 0) sms = fmx_num_sms();
  return (wide < 32 && (n_out + wide - 1) / wide < sms && K >= 4096) ? 16 : 8;
}


// x [M <= 16, K] and W [N, K] bfloat16, rows 16-byte aligned; out [M, N] bfloat16 (out_dtype 1)
// or float (0); bias float[N] or null; residual bfloat16 [M, n_out] or null (may be `out`).
// blk > 0: W's rows alternate in blocks of blk gate rows and blk up rows, out is [M, N/2] =
// silu(gate) * up in bfloat16.  wide: 8, 16 or 32 output features per block; warps: 8 or 16
// per block (16 when few blocks must keep many bytes in flight over a long K).
FMX_EXPORT int fmx_gemv(const void* x, long long ldx, const void* W, long long ldw, const float* bias, const void* residual,
                        long long ldr, void* out, long long ldo, int M, int N, int K, int out_dtype, int blk, int wide,
                        int warps, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || M > 16 || N < 0 || K <= 0) return fmx_fail("fmx_gemv: takes 1..16 rows, got M=%d N=%d K=%d", M, N, K);
  if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x & 15) || ((uintptr_t)W & 15))
    return fmx_fail("fmx_gemv: rows must be 16-byte aligned (K=%d ldx=%lld ldw=%lld)", K, ldx, ldw);
  if (blk < 0 || (blk > 0 && (blk % 16 || N % (2 * blk))))
    return fmx_fail("fmx_gemv: gate/up blocks of %d do not tile %d rows", blk, N);
  if (blk > 0 && out_dtype != FMX_BF16) return fmx_fail("fmx_gemv: the SiLU-mul epilogue writes bfloat16");
  const bool hi = M > 8;
  const int n_out = blk > 0 ? N / 2 : N;
  if (wide == 0) wide = fmx_gemv_plan_width(n_out, blk, 0);
  if (warps == 0) warps = fmx_gemv_plan_warps(n_out, K, wide, 0);
  if (warps != 8 && warps != 16) return fmx_fail("fmx_gemv: 8 or 16 warps per block, not %d", warps);
  if (warps == 16 && wide == 32) return fmx_fail("fmx_gemv: 32 features per block go with 8 warps");
  if (wide != 8 && wide != 16 && wide != 32) return fmx_fail("fmx_gemv: 8, 16 or 32 features per block, not %d", wide);
  if (blk > 0 && blk % wide) return fmx_fail("fmx_gemv: %d features per block do not tile gate/up blocks of %d", wide, blk);
#define FMX_GV1(NT_, HI_, DUAL_, U_, W_, TO_) \
  launch<NT_, HI_, DUAL_, U_, W_, TO_>(x, ldx, W, ldw, bias, residual, ldr, out, ldo, M, N, K, blk, stream)
#define FMX_GV(NT_, HI_, DUAL_, U_, TO_)                 \
  do {                                                   \
    if (warps == 16) FMX_GV1(NT_, HI_, DUAL_, U_, 16, TO_); \
    else FMX_GV1(NT_, HI_, DUAL_, U_, 8, TO_);           \
  } while (0)
#define FMX_GV_WIDTHS(HI_, DUAL_, TO_, U8, U16, U32)      \
  do {                                                    \
    if (wide == 8) FMX_GV(1, HI_, DUAL_, U8, TO_);        \
    else if (wide == 16) FMX_GV(2, HI_, DUAL_, U16, TO_); \
    else FMX_GV1(4, HI_, DUAL_, U32, 8, TO_);             \
  } while (0)
  if (blk > 0) {
    if (hi) FMX_GV_WIDTHS(true, true, bf16, 4, 2, 1);
    else FMX_GV_WIDTHS(false, true, bf16, 8, 4, 2);
  } else if (out_dtype == FMX_BF16) {
    if (hi) FMX_GV_WIDTHS(true, false, bf16, 8, 4, 2);
    else FMX_GV_WIDTHS(false, false, bf16, 8, 8, 4);
  } else if (out_dtype == FMX_F32) {
    if (hi) FMX_GV_WIDTHS(true, false, float, 8, 4, 2);
    else FMX_GV_WIDTHS(false, false, float, 8, 8, 4);
  } else {
    return fmx_fail("fmx_gemv: unknown output dtype %d", out_dtype);
  }
#undef FMX_GV_WIDTHS
#undef FMX_GV1
#undef FMX_GV
  FMX_LAUNCH_CHECK();
  return 0;
}
