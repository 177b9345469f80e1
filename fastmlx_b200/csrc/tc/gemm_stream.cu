// out[M, N] = x[M, K] . W[N, K]^T for few rows (M <= 128): the products of a decode step,
// which are bound by streaming W from HBM once.  The operands are swapped: a tile of 128 rows
// of W is the A operand of tcgen05.mma (one output feature per lane of tensor memory), the
// rows of x are the B operand (one token per column).  W never passes through registers:
// TMA brings it into a ring of shared-memory stages, one thread issues the MMAs, and four
// warps read the finished accumulators back with tcgen05.ld.
//
// Work is dealt out stream-K fashion.  A unit is one stage: 128 rows of W x 128 of K (two
// 16 KB boxes; for a gate/up pair 256 rows x 64 of K), eight MMAs: the thread that issues
// them spends some 60 cycles on each and as much again per stage on its barrier and commit,
// so a stage must carry enough bytes for that thread to keep up with HBM.  The n_tiles x k_blocks units are numbered tile-major and cut
// into gridDim.x equal contiguous ranges, one per CTA, whatever the matrix's shape: every SM
// streams the same number of bytes.  A range may start and end in the middle of a tile; such
// a partial sum goes to a workspace slot, the CTA takes a ticket of the tile, and the CTA
// that draws a tile's last ticket adds the partials in CTA order and writes the result.
// Nobody waits for anybody, and the order of the sum is fixed.
//
// Under programmatic dependent launch the producer fills the whole ring with W before it
// waits for the kernel ahead (W is never written by a kernel); only the loads of x come
// after the wait.  With about 100 KB of ring a CTA fits beside a CTA of the kernel ahead, so
// that the weights of a small product are already in shared memory when its input is ready.
//
// Epilogues: plain (+ bias, bfloat16 or float out); SiLU(gate) * up for a weight whose rows
// alternate in blocks of 128 gate rows and their 128 up rows (both halves of a pair are
// accumulated side by side in tensor memory).
//
// Every wait on a barrier is bounded by time; a wait that expires leaves FMX_WAIT_EXPIRED in
// the status word, and the CTA drains its copies in flight, frees its tensor memory and returns.
#include <cuda.h>
#include "common.cuh"
#include "tcgen05.cuh"

namespace {
using namespace fmx_tc;
constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int EPI_THREADS = 128;

__device__ __host__ __forceinline__ long long range_start(long long c, long long total, long long ctas) {
  return c * total / ctas;
}

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int HALVES, typename TO>                  // HALVES = 2: gate and up tiles of one pair
__global__ void __launch_bounds__(THREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TO* out,
                   long long ldo, const float* __restrict__ bias, int M, int N, int K, int NB, int stages, float* ws,
                   int* tickets, int* status) {
  constexpr int KSUB = HALVES == 2 ? 1 : 2;         // 64-wide k blocks per stage
  constexpr int A_BYTES = HALVES * BM * BK * 2;     // one k block of W
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int x_bytes = NB * BK * 2, sub_bytes = A_BYTES + x_bytes, stage_bytes = KSUB * sub_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)stages * stage_bytes);
  uint64_t* full_bar = bars;                       // [stages]
  uint64_t* empty_bar = bars + stages;             // [stages]
  uint64_t* acc_full = bars + 2 * stages;          // [2]
  uint64_t* acc_empty = acc_full + 2;              // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  int* epi_flag = reinterpret_cast<int*>(tmem_slot + 1);      // [0] a wait expired, [1] the ticket drawn

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = HALVES == 2 ? N / (2 * BM) : (N + BM - 1) / BM;
  const int kb = (K + KSUB * BK - 1) / (KSUB * BK);
  const long long total = (long long)n_tiles * kb;
  const long long s0 = range_start(blockIdx.x, total, gridDim.x), s1 = range_start(blockIdx.x + 1, total, gridDim.x);
  const int n_units = (int)(s1 - s0), tile0 = (int)(s0 / kb), k0 = (int)(s0 - (long long)tile0 * kb);
  const int acc_cols = HALVES * NB;                // columns of one accumulator
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < 2 * acc_cols) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&acc_full[a]), 1);
      mbar_init(smem_u32(&acc_empty[a]), EPI_THREADS);
    }
    epi_flag[0] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    int issued = 0;
    bool ok = true;
    const int ahead = min(stages, n_units);
    // (tile, k) of a unit advance by counting: a 64-bit division per unit would cost more
    // than the unit's copy.
    int tile = tile0, k = k0;
    // The ring is empty: W of the first units goes out before the kernel ahead has finished.
    for (int st = 0; st < ahead; ++st) {
      const uint32_t fb = smem_u32(&full_bar[st]);
      mbar_expect_tx(fb, (uint32_t)stage_bytes);
#pragma unroll
      for (int j = 0; j < KSUB; ++j)
        tma_load_2d(smem_u32(smem + (size_t)st * stage_bytes + j * sub_bytes), &map_w, (k * KSUB + j) * BK,
                    tile * HALVES * BM, fb);
      if (++k == kb) { k = 0; ++tile; }
    }
    pdl_wait();                                    // x is the output of the kernel ahead
    pdl_trigger();
    for (int st = 0, kx = k0; st < ahead; ++st) {
#pragma unroll
      for (int j = 0; j < KSUB; ++j)
        tma_load_2d(smem_u32(smem + (size_t)st * stage_bytes + j * sub_bytes + A_BYTES), &map_x, (kx * KSUB + j) * BK, 0,
                    smem_u32(&full_bar[st]));
      if (++kx == kb) kx = 0;
    }
    issued = ahead;
    stage = ahead % stages;
    phase = ahead == stages ? 1u : 0u;
    for (int u = ahead; u < n_units; ++u) {
      if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1)) { ok = false; break; }
      const uint32_t fb = smem_u32(&full_bar[stage]);
      unsigned char* sa = smem + (size_t)stage * stage_bytes;
      mbar_expect_tx(fb, (uint32_t)stage_bytes);
#pragma unroll
      for (int j = 0; j < KSUB; ++j) {
        tma_load_2d(smem_u32(sa + j * sub_bytes), &map_w, (k * KSUB + j) * BK, tile * HALVES * BM, fb);
        tma_load_2d(smem_u32(sa + j * sub_bytes + A_BYTES), &map_x, (k * KSUB + j) * BK, 0, fb);
      }
      ++issued;
      if (++stage == stages) { stage = 0; phase ^= 1; }
      if (++k == kb) { k = 0; ++tile; }
    }
    if (!ok) {
      fmx_set_status(status, FMX_WAIT_EXPIRED, 1, blockIdx.x);
      const int pending = issued < stages ? issued : stages;
      for (int s = 0; s < pending; ++s) mbar_wait(smem_u32(&full_bar[s]), 0) || mbar_wait(smem_u32(&full_bar[s]), 1);
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc = make_idesc(BM, NB);
    int stage = 0, acc = 0;
    uint32_t phase = 0, acc_phase = 0;
    bool ok = true;
    pdl_wait();                                    // so that the bounded waits below start when the input exists
    int k = k0;
    for (int u = 0; u < n_units && ok; ++u) {
      const bool first = u == 0 || k == 0, last = u == n_units - 1 || k == kb - 1;
      if (++k == kb) k = 0;
      if (first) {
        if (!mbar_wait(smem_u32(&acc_empty[acc]), acc_phase ^ 1)) { ok = false; break; }
        tc_fence_after();
      }
      if (!mbar_wait(smem_u32(&full_bar[stage]), phase)) { ok = false; break; }
      tc_fence_after();
      const uint32_t sa = smem_u32(smem + (size_t)stage * stage_bytes);
#pragma unroll
      for (int sub = 0; sub < KSUB; ++sub) {
        const uint64_t bdesc = make_desc_k128(sa + sub * sub_bytes + A_BYTES);
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
          const uint64_t adesc = make_desc_k128(sa + sub * sub_bytes + h * BM * BK * 2);
          const uint32_t tmem_d = tmem_base + (uint32_t)(acc * acc_cols + h * NB);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j)
            umma_f16(tmem_d, adesc + 2 * j, bdesc + 2 * j, idesc, (!first || sub > 0 || j > 0) ? 1u : 0u);
        }
      }
      umma_commit(smem_u32(&empty_bar[stage]));
      if (++stage == stages) { stage = 0; phase ^= 1; }
      if (last) {
        umma_commit(smem_u32(&acc_full[acc]));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    if (!ok) fmx_set_status(status, FMX_WAIT_EXPIRED, 2, blockIdx.x);
  } else if (warp >= 2) {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;                  // the 32 lanes of tensor memory this warp may read
    const int row = quarter * 32 + lane;           // output feature within the tile
    const int etid = threadIdx.x - 64;
    const int n_out = HALVES == 2 ? N / 2 : N;
    const long long slot_floats = (long long)HALVES * M * BM;
    int acc = 0;
    uint32_t acc_phase = 0;
    pdl_wait();                                    // before the first write anything ahead may still read
    long long s = s0;
    int tile = tile0, k_first = k0;
    while (s < s1) {
      const long long seg_end = min(s1, (long long)(tile + 1) * kb);
      const bool whole = k_first == 0 && seg_end == (long long)(tile + 1) * kb;
      const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&acc_full[acc]), acc_phase));   // warp-uniform
      if (!ok) epi_flag[0] = 1;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * acc_cols);
      const int n = tile * BM + row;                // output column this thread owns
      // the CTA's first segment uses slot 0, its last (if another) slot 1
      float* mine = ws + ((long long)blockIdx.x * 2 + (s == s0 ? 0 : 1)) * slot_floats;
      for (int c = 0; c < M && ok; c += 16) {
        uint32_t v[16], u[16];
        tmem_ld16(taddr + c, v);
        if (HALVES == 2) tmem_ld16(taddr + NB + c, u);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int tok = c + i;
          if (tok >= M) break;
          if (whole) {
            if (n < n_out) {
              float r = __uint_as_float(v[i]);
              if (HALVES == 2) {
                const float g = bf16r(r);
                r = g / (1.0f + expf(-g)) * bf16r(__uint_as_float(u[i]));
              } else if (bias != nullptr) {
                r += bias[n];
              }
              store_out<TO>(out + (long long)tok * ldo + n, r);
            }
          } else {
            __stcg(mine + (long long)tok * BM + row, __uint_as_float(v[i]));
            if (HALVES == 2) __stcg(mine + (long long)(M + tok) * BM + row, __uint_as_float(u[i]));
          }
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&acc_empty[acc]));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      if (!whole) __threadfence();
      epi_bar();
      if (epi_flag[0]) break;                      // all four warps leave together
      if (!whole) {
        // contributors of this tile: the CTAs whose ranges meet [tile * kb, (tile + 1) * kb)
        const long long t0 = (long long)tile * kb, t1 = t0 + kb - 1;
        long long c_lo = (t0 + 1) * gridDim.x / total, c_hi = (t1 + 1) * gridDim.x / total;
        if (c_lo >= gridDim.x) c_lo = gridDim.x - 1;
        if (c_hi >= gridDim.x) c_hi = gridDim.x - 1;
        while (c_lo > 0 && range_start(c_lo, total, gridDim.x) > t0) --c_lo;
        while (c_lo + 1 < gridDim.x && range_start(c_lo + 1, total, gridDim.x) <= t0) ++c_lo;
        while (c_hi > 0 && range_start(c_hi, total, gridDim.x) > t1) --c_hi;
        while (c_hi + 1 < gridDim.x && range_start(c_hi + 1, total, gridDim.x) <= t1) ++c_hi;
        if (etid == 0) epi_flag[1] = atomicAdd(&tickets[tile], 1);
        epi_bar();
        const bool reducer = epi_flag[1] == (int)(c_hi - c_lo);
        epi_bar();                                 // the flag is free for the next segment
        if (reducer) {
          __threadfence();
          if (n < n_out) {
            // of the contributors only the lowest may have begun before this tile (its slot 1)
            const bool lo_first = range_start(c_lo, total, gridDim.x) >= t0;
            for (int tk = 0; tk < M; tk += 8) {
              float g[8], w[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) g[i] = w[i] = 0.f;
              for (long long c = c_lo; c <= c_hi; ++c) {
                const float* p = ws + (c * 2 + ((c > c_lo || lo_first) ? 0 : 1)) * slot_floats + row;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  if (tk + i < M) {
                    g[i] += __ldcg(p + (long long)(tk + i) * BM);
                    if (HALVES == 2) w[i] += __ldcg(p + (long long)(M + tk + i) * BM);
                  }
                }
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                if (tk + i >= M) break;
                float r = g[i];
                if (HALVES == 2) {
                  const float gg = bf16r(g[i]);
                  r = gg / (1.0f + expf(-gg)) * bf16r(w[i]);
                } else if (bias != nullptr) {
                  r += bias[n];
                }
                store_out<TO>(out + (long long)(tk + i) * ldo + n, r);
              }
            }
          }
          if (etid == 0) tickets[tile] = 0;         // ready for the next launch
        }
      }
      s = seg_end;
      ++tile;
      k_first = 0;
    }
    if (epi_flag[0] && etid == 0) fmx_set_status(status, FMX_WAIT_EXPIRED, 3, blockIdx.x);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

template <int HALVES, typename TO>
int run(const CUtensorMap& map_w, const CUtensorMap& map_x, void* out, long long ldo, const float* bias, int M, int N,
        int K, int NB, int stages, int ctas, float* ws, int* tickets, int* status, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<HALVES, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         227 * 1024);
    if (e != cudaSuccess) return fmx_fail("gemm_stream: shared memory refused: %s", cudaGetErrorString(e));
    configured = true;
  }
  const size_t smem = (size_t)stages * (32768 + (HALVES == 2 ? 1 : 2) * NB * BK * 2) + 1024 + 16 * (size_t)stages + 64;
  cudaError_t e = fmx_launch(gemm_stream_kernel<HALVES, TO>, dim3(ctas), dim3(THREADS), smem, stream, map_w, map_x,
                             (TO*)out, ldo, bias, M, N, K, NB, stages, ws, tickets, status);
  if (e != cudaSuccess) return fmx_fail("gemm_stream: launch failed: %s", cudaGetErrorString(e));
  return 0;
}

int columns_for(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128; }
}  // namespace

// x [M <= 128, K] and W [N, K] bfloat16, K-contiguous rows starting on 16-byte boundaries;
// out [M, N] bfloat16 (out_dtype 1) or float (0), or [M, N/2] = silu(gate) * up when dual.
// ctas: at most one per unit of 128 rows x 128 of K (dual: 256 x 64); stages: the ring's depth.
// ws: ctas * 2 * (dual ? 2 : 1) * M * 128 floats of partial sums; tickets: one per tile, zero
// before the first call (every call leaves them zero).  Calls that share them must not overlap
// on the GPU.
FMX_EXPORT int fmx_gemm_stream(const void* x, long long ldx, const void* W, long long ldw, const float* bias, void* out,
                               long long ldo, int M, int N, int K, int out_dtype, int dual, int ctas, int stages,
                               float* ws, long long ws_floats, int* tickets, long long n_tickets, int* status,
                               cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || M > 128 || N < 0 || K <= 0) return fmx_fail("fmx_gemm_stream: takes 1..128 rows, got M=%d N=%d K=%d", M, N, K);
  if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x & 15) || ((uintptr_t)W & 15))
    return fmx_fail("fmx_gemm_stream: rows must start on 16-byte boundaries (K=%d ldx=%lld ldw=%lld)", K, ldx, ldw);
  const int halves = dual ? 2 : 1;
  if (dual && N % (2 * BM)) return fmx_fail("fmx_gemm_stream: gate/up pairs of 2 x %d rows do not tile %d rows", BM, N);
  if (dual && (out_dtype != FMX_BF16 || bias != nullptr))
    return fmx_fail("fmx_gemm_stream: the SiLU-mul epilogue writes bfloat16 and takes no bias");
  const int NB = columns_for(M);
  const int ksub = dual ? 1 : 2;
  const long long tiles = dual ? N / (2 * BM) : (N + BM - 1) / BM, kb = (K + ksub * BK - 1) / (ksub * BK);
  const long long total = tiles * kb;
  if (ctas < 1 || ctas > total) return fmx_fail("fmx_gemm_stream: %d CTAs for %lld units", ctas, total);
  const long long stage_bytes = 32768 + ksub * NB * BK * 2;
  if (stages < 2 || stages * stage_bytes + 2048 > 227 * 1024) return fmx_fail("fmx_gemm_stream: bad stage count %d", stages);
  if (ws == nullptr || tickets == nullptr || ws_floats < (long long)ctas * 2 * halves * M * BM || n_tickets < tiles)
    return fmx_fail("fmx_gemm_stream: needs %lld floats of workspace and %lld tickets", (long long)ctas * 2 * halves * M * BM,
                    tiles);
  CUtensorMap map_w, map_x;
  if (make_map_k128(&map_w, W, N, K, ldw, halves * BM) || make_map_k128(&map_x, x, M, K, ldx, NB)) return 1;
#define FMX_GS(H_, TO_) return run<H_, TO_>(map_w, map_x, out, ldo, bias, M, N, K, NB, stages, ctas, ws, tickets, status, stream)
  if (dual) FMX_GS(2, bf16);
  if (out_dtype == FMX_BF16) FMX_GS(1, bf16);
  if (out_dtype == FMX_F32) FMX_GS(1, float);
#undef FMX_GS
  return fmx_fail("fmx_gemm_stream: unknown output dtype %d", out_dtype);
}
