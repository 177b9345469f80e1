// out[M, N] = x[M, K] . W[N, K]^T for a handful of rows (M <= 16): the matrix products of a
// decode step, which are bound by streaming W from HBM once.
//
// W is the A operand of mma.sync m16n8k16 (16 output features per block), x the B operand
// (8 tokens per column tile).  No shared-memory staging: the sum over k does not care in
// which order k is visited, so each thread loads 16 contiguous bytes of a W row (and of an
// x row) straight into registers and hands them to two MMAs under a fixed permutation of k
// that is the same for both operands.  The eight warps of a block take interleaved 32-wide
// slices of K, so that together they read 512 contiguous bytes of each row, and their
// partial sums are added in a fixed order at the end.
//
// When N is small the grid would leave most SMs idle, so K can also be split over blocks
// (gridDim.y): each block leaves its partial tile in a workspace and takes a ticket; the
// block that draws the last ticket of a tile adds the partials in split order and writes
// the result.  Nobody waits for anybody, and the sum's order is fixed.
//
// Up to eight splits can instead form a thread-block cluster (gridDim.y = the cluster's size):
// every block leaves its partial tile in its own shared memory, and after one cluster barrier
// the block of rank 0 reads its peers' tiles through distributed shared memory, in rank order.
// That replaces a store, a fence, an atomic and a load through L2 by one hardware barrier.
#include "common.cuh"

namespace {
constexpr int WARPS = 8;

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_peer(const float* mine, unsigned rank) {
  unsigned a = (unsigned)__cvta_generic_to_shared(mine), ra;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
  return v;
}

template <int MT, int U, typename TO, bool CLUSTER>
__global__ void __launch_bounds__(WARPS * 32)
skinny_gemm_kernel(const bf16* x, long long ldx, const bf16* __restrict__ W, long long ldw,
                   const float* __restrict__ bias, TO* __restrict__ out, long long ldo, int M, int N, int K,
                   float* __restrict__ ws, int* __restrict__ tickets) {
  __shared__ float red[WARPS][16][8 * MT + 1];
  __shared__ int last_ticket;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  const bf16* w0 = W + (long long)min(n0 + g, N - 1) * ldw + 8 * t;
  const bf16* w1 = W + (long long)min(n0 + g + 8, N - 1) * ldw + 8 * t;
  const bf16* xp[MT];
  bool xok[MT];
#pragma unroll
  for (int j = 0; j < MT; ++j) {
    xok[j] = 8 * j + g < M;
    xp[j] = x + (long long)(xok[j] ? 8 * j + g : 0) * ldx + 8 * t;
  }
  float acc[MT][4];
#pragma unroll
  for (int j = 0; j < MT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  const int nkb_all = (K + 31) / 32;
  const int per_split = (nkb_all + gridDim.y - 1) / gridDim.y;
  const int kb0 = blockIdx.y * per_split;
  const int nkb = min(nkb_all, kb0 + per_split);
  bool waited = false;
  for (int kb = kb0 + warp; kb < nkb; kb += WARPS * U) {
    uint4 a0[U], a1[U], b[U][MT];
    // W is never written by a kernel: its first loads go out before the wait for the
    // predecessor, whose output x is.  x must not be read through the read-only path
    // (__ldg, or a __restrict__ const pointer): the compiler may move such a load above
    // the wait, where x is still being written.
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (kb + WARPS * u) * 32;
      const bool ok = kb + WARPS * u < nkb && k + 8 * t < K;    // K is a multiple of 8: all 16 bytes or none
      a0[u] = ok ? __ldcs(reinterpret_cast<const uint4*>(w0 + k)) : zero;
      a1[u] = ok ? __ldcs(reinterpret_cast<const uint4*>(w1 + k)) : zero;
    }
    if (!waited) {
      pdl_wait();
      pdl_trigger();
      waited = true;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (kb + WARPS * u) * 32;
      const bool ok = kb + WARPS * u < nkb && k + 8 * t < K;
#pragma unroll
      for (int j = 0; j < MT; ++j) b[u][j] = (ok && xok[j]) ? __ldcg(reinterpret_cast<const uint4*>(xp[j] + k)) : zero;
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        mma_bf16(acc[j], a0[u].x, a1[u].x, a0[u].y, a1[u].y, b[u][j].x, b[u][j].y);
        mma_bf16(acc[j], a0[u].z, a1[u].z, a0[u].w, a1[u].w, b[u][j].z, b[u][j].w);
      }
  }
  if (!waited) {
    pdl_wait();
    pdl_trigger();
  }                             // a warp without a k block still orders its writes
#pragma unroll
  for (int j = 0; j < MT; ++j) {
    red[warp][g][8 * j + 2 * t] = acc[j][0];
    red[warp][g][8 * j + 2 * t + 1] = acc[j][1];
    red[warp][g + 8][8 * j + 2 * t] = acc[j][2];
    red[warp][g + 8][8 * j + 2 * t + 1] = acc[j][3];
  }
  __syncthreads();
  constexpr int TILE_ELEMS = 16 * 8 * MT;
  const int splits = gridDim.y;
  if (CLUSTER) {
    __shared__ float part[TILE_ELEMS];
    for (int idx = threadIdx.x; idx < TILE_ELEMS; idx += WARPS * 32) {
      const int tok = idx / 16, row = idx - tok * 16;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) v += red[w][row][tok];
      part[idx] = v;
    }
    cluster_sync();                                      // every block's tile is in its shared memory
    if (blockIdx.y == 0) {
      for (int idx = threadIdx.x; idx < TILE_ELEMS; idx += WARPS * 32) {
        const int tok = idx / 16, row = idx - tok * 16;
        const int n = n0 + row;
        if (tok >= M || n >= N) continue;
        float v = 0.f;
        for (int sp = 0; sp < splits; ++sp) v += ld_peer(part + idx, (unsigned)sp);
        if (bias) v += bias[n];
        store_out<TO>(out + (long long)tok * ldo + n, v);
      }
    }
    cluster_sync();                                      // nobody leaves while its tile may still be read
    return;
  }
  if (splits == 1) {
    for (int idx = threadIdx.x; idx < TILE_ELEMS; idx += WARPS * 32) {
      const int tok = idx / 16, row = idx - tok * 16;    // consecutive threads write consecutive features
      const int n = n0 + row;
      if (tok >= M || n >= N) continue;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) v += red[w][row][tok];
      if (bias) v += bias[n];
      store_out<TO>(out + (long long)tok * ldo + n, v);
    }
    return;
  }
  float* mine = ws + ((long long)blockIdx.x * splits + blockIdx.y) * TILE_ELEMS;
  for (int idx = threadIdx.x; idx < TILE_ELEMS; idx += WARPS * 32) {
    const int tok = idx / 16, row = idx - tok * 16;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) v += red[w][row][tok];
    __stcg(mine + idx, v);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last_ticket = atomicAdd(&tickets[blockIdx.x], 1);
  __syncthreads();
  if (last_ticket != splits - 1) return;
  __threadfence();
  const float* all = ws + (long long)blockIdx.x * splits * TILE_ELEMS;
  for (int idx = threadIdx.x; idx < TILE_ELEMS; idx += WARPS * 32) {
    const int tok = idx / 16, row = idx - tok * 16;
    const int n = n0 + row;
    if (tok >= M || n >= N) continue;
    float v = 0.f;
    for (int sp = 0; sp < splits; ++sp) v += __ldcg(all + (long long)sp * TILE_ELEMS + idx);
    if (bias) v += bias[n];
    store_out<TO>(out + (long long)tok * ldo + n, v);
  }
  if (threadIdx.x == 0) tickets[blockIdx.x] = 0;          // ready for the next launch
}

template <int MT, int U, typename TO>
void launch(const void* x, long long ldx, const void* W, long long ldw, const float* bias, void* out, long long ldo,
            int M, int N, int K, int splits, float* ws, int* tickets, bool cluster, cudaStream_t stream) {
  if (cluster)
    fmx_launch_cluster(skinny_gemm_kernel<MT, U, TO, true>, dim3((N + 15) / 16, splits), dim3(WARPS * 32), 0, stream,
                       dim3(1, splits, 1), (const bf16*)x, ldx, (const bf16*)W, ldw, bias, (TO*)out, ldo, M, N, K, ws,
                       tickets);
  else
    fmx_launch(skinny_gemm_kernel<MT, U, TO, false>, dim3((N + 15) / 16, splits), dim3(WARPS * 32), 0, stream,
               (const bf16*)x, ldx, (const bf16*)W, ldw, bias, (TO*)out, ldo, M, N, K, ws, tickets);
}
}  // namespace

// Floats of workspace and ints of tickets a call with `splits` > 1 needs.  The tickets must
// be zero before the first call; every call leaves them zero again.  Calls that share a
// workspace must not overlap on the GPU.
FMX_EXPORT long long fmx_skinny_gemm_ws_floats(int M, int N, int splits) {
  return splits <= 1 ? 0 : (long long)((N + 15) / 16) * splits * 16 * 8 * (M <= 8 ? 1 : 2);
}
FMX_EXPORT long long fmx_skinny_gemm_tickets(int N, int splits) { return splits <= 1 ? 0 : (N + 15) / 16; }

// x, W bfloat16 with rows 16-byte aligned (K, ldx, ldw multiples of 8); out bfloat16
// (out_dtype 1) or float (0); bias float or null.  splits < 0: -splits blocks (2..8) form a
// cluster and reduce through distributed shared memory; no workspace is used.
FMX_EXPORT int fmx_skinny_gemm(const void* x, long long ldx, const void* W, long long ldw, const float* bias, void* out,
                               long long ldo, int M, int N, int K, int out_dtype, int splits, float* ws,
                               long long ws_floats, int* tickets, long long n_tickets, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || M > 16 || N < 0 || K <= 0) return fmx_fail("fmx_skinny_gemm: takes 1..16 rows, got M=%d N=%d K=%d", M, N, K);
  if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x & 15) || ((uintptr_t)W & 15))
    return fmx_fail("fmx_skinny_gemm: rows must be 16-byte aligned (K=%d ldx=%lld ldw=%lld)", K, ldx, ldw);
  const bool cluster = splits < 0;
  if (cluster) splits = -splits;
  if (cluster && (splits < 2 || splits > 8)) return fmx_fail("fmx_skinny_gemm: a cluster holds 2..8 splits, not %d", splits);
  if (splits < 1 || splits > 65535) return fmx_fail("fmx_skinny_gemm: bad split count %d", splits);
  if (splits > 1 && !cluster && (ws == nullptr || tickets == nullptr || ws_floats < fmx_skinny_gemm_ws_floats(M, N, splits) ||
                     n_tickets < fmx_skinny_gemm_tickets(N, splits)))
    return fmx_fail("fmx_skinny_gemm: %d splits need %lld floats and %lld tickets of workspace", splits,
                    fmx_skinny_gemm_ws_floats(M, N, splits), fmx_skinny_gemm_tickets(N, splits));
  if (out_dtype == FMX_BF16) {
    if (M <= 8) launch<1, 8, bf16>(x, ldx, W, ldw, bias, out, ldo, M, N, K, splits, ws, tickets, cluster, stream);
    else launch<2, 4, bf16>(x, ldx, W, ldw, bias, out, ldo, M, N, K, splits, ws, tickets, cluster, stream);
  } else if (out_dtype == FMX_F32) {
    if (M <= 8) launch<1, 8, float>(x, ldx, W, ldw, bias, out, ldo, M, N, K, splits, ws, tickets, cluster, stream);
    else launch<2, 4, float>(x, ldx, W, ldw, bias, out, ldo, M, N, K, splits, ws, tickets, cluster, stream);
  } else {
    return fmx_fail("fmx_skinny_gemm: unknown output dtype %d", out_dtype);
  }
  FMX_LAUNCH_CHECK();
  return 0;
}
