// C[M, N] = A[M, K] . W[N, K]^T in bfloat16 with 32-bit accumulation on the fifth-generation
// tensor cores: tcgen05.mma issued by one thread, operands staged in shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), accumulators in tensor memory and read back with
// tcgen05.ld for the epilogue.  This is the matrix product of prefill steps.
//
// One persistent CTA per SM walks over 128 x BN output tiles.  Six warps, three roles:
//   warp 0, one lane : producer.  Waits for a free stage, arms its "full" barrier with the
//                      stage's byte count and issues two TMA loads (A tile 128 x 64, W tile
//                      BN x 64).  Both operands are K-major, so one box is one 128-byte row
//                      per matrix row: exactly the canonical SWIZZLE_128B layout the MMA reads.
//   warp 1, one lane : MMA issuer.  Waits for a full stage, issues four 128 x BN x 16 MMAs
//                      (advancing the descriptors by 32 bytes along K), commits to the stage's
//                      "empty" barrier; after the last k block commits to the accumulator's
//                      "full" barrier.  Two accumulators in tensor memory let the next tile's
//                      mainloop run under this tile's epilogue.
//   warps 2-5        : epilogue.  Each warp owns the 32 lanes of tensor memory it may read
//                      (warp index mod 4), loads 16 columns at a time, converts and stores.
//                      Variants: plain; SiLU(gate) * up for a weight whose rows come in blocks
//                      of BN/2 gate rows followed by their BN/2 up rows; residual add.
//
// No cluster: every CTA loads its own tiles.  Every wait on a barrier is bounded by time: after about a
// second it gives up, leaves FMX_WAIT_EXPIRED in the status word, and the CTA drains what it
// has in flight, frees its tensor memory and returns.
//
// Compiled with -DFMX_SKIP_LAST_STAGE (and a short -DFMX_WAIT_CYCLES) the producer leaves out the
// last k block of its CTA's last tile: the issuing thread and the epilogue warps then wait for
// something that never comes, with no copy in flight, and the expiry path runs.  Only the test
// library `tc_expiry` is built that way; the product library never is.
#include <cuda.h>
#include "common.cuh"
#include "tcgen05.cuh"

namespace {
using namespace fmx_tc;
constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int THREADS = 192;

enum Epilogue { EPI_PLAIN = 0, EPI_SILU_MUL = 1, EPI_RESIDUAL = 2 };

template <int BN> struct Cfg {
  static constexpr int STAGES = BN == 256 ? 4 : (BN == 192 ? 5 : 6);
  static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = BN > 128 ? 512 : 256;   // two accumulators; a power of two >= 32
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /* alignment */ + 256 /* barriers */;
  static_assert((2 * STAGES + 5) * 8 + 4 <= 256, "the barriers outgrow their corner of shared memory");
};

__device__ __forceinline__ unsigned pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float silu(float g) { return g / (1.0f + expf(-g)); }

template <int BN, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, bf16* C,
                    long long ldc, const bf16* residual, long long ldr, int M, int N, int K, int* status) {
  using cfg = Cfg<BN>;
  extern __shared__ unsigned char smem_raw[];
  // 1024-byte alignment: the swizzle pattern repeats every eight 128-byte rows
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)cfg::STAGES * cfg::STAGE_BYTES);
  uint64_t* full_bar = bars;                       // [STAGES]
  uint64_t* empty_bar = bars + cfg::STAGES;        // [STAGES]
  uint64_t* acc_full = bars + 2 * cfg::STAGES;     // [2]
  uint64_t* acc_empty = acc_full + 2;              // [2]
  uint64_t* drain_bar = acc_empty + 2;             // [1] a wait that expired: have the products issued so far finished?
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < cfg::STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&acc_full[a]), 1);
      mbar_init(smem_u32(&acc_empty[a]), 128);
    }
    mbar_init(smem_u32(drain_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(cfg::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                                      // A is the output of the kernel before this one
  pdl_trigger();

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    long long issued = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
      const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
      for (int kb = 0; kb < k_blocks; ++kb) {
#ifdef FMX_SKIP_LAST_STAGE
        if (kb == k_blocks - 1 && t + (int)gridDim.x >= n_tiles) break;      // the test build: never bring the last block
#endif
        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1)) { ok = false; break; }
        const uint32_t fb = smem_u32(&full_bar[stage]);
        unsigned char* sa = smem + (size_t)stage * cfg::STAGE_BYTES;
        mbar_expect_tx(fb, cfg::STAGE_BYTES);
        tma_load_2d(smem_u32(sa), &map_a, kb * BK, m0, fb);
        tma_load_2d(smem_u32(sa + cfg::A_BYTES), &map_w, kb * BK, n0, fb);
        ++issued;
        if (++stage == cfg::STAGES) { stage = 0; phase ^= 1; }
      }
    }
    if (!ok) {
      fmx_set_status(status, FMX_WAIT_EXPIRED, 1, blockIdx.x);
      // its own copies in flight: give each armed stage a bounded chance to land
      const int pending = (int)(issued < cfg::STAGES ? issued : cfg::STAGES);
      for (int s = 0; s < pending; ++s) mbar_wait(smem_u32(&full_bar[s]), 0) || mbar_wait(smem_u32(&full_bar[s]), 1);
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------ MMA issuer
    // Whatever this thread executes between two products is time the tensor pipe stands still
    // (a measured 128 x 256 x 16 product takes 128 clocks back to back, 171 with a dozen
    // instructions of descriptor arithmetic in between).  So the walk over the ring is unrolled by
    // the number of stages: each stage's descriptors and barrier addresses are built once, before
    // the loop, and tile borders are a counter inside it.
    const uint32_t idesc = make_idesc(BM, BN);
    uint32_t a_lo[cfg::STAGES], b_lo[cfg::STAGES];
#pragma unroll
    for (int s = 0; s < cfg::STAGES; ++s) {
      const uint32_t sa = smem_u32(smem + (size_t)s * cfg::STAGE_BYTES);
      a_lo[s] = (uint32_t)make_desc_k128(sa);
      b_lo[s] = (uint32_t)make_desc_k128(sa + cfg::A_BYTES);
    }
    const uint64_t desc_hi = make_desc_k128(0) & 0xffffffff00000000ull;
    const int my_tiles = blockIdx.x < n_tiles ? (n_tiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    const long long total = (long long)my_tiles * k_blocks;
    int acc = 0, kb = 0;
    uint32_t phase = 0, acc_phase = 0, tmem_d = tmem_base;
    bool ok = true;
    for (long long g = 0; g < total && ok; g += cfg::STAGES) {
#pragma unroll
      for (int s = 0; s < cfg::STAGES; ++s) {
        if (g + s >= total || !ok) break;
        if (kb == 0) {
          if (!mbar_wait(smem_u32(&acc_empty[acc]), acc_phase ^ 1)) { ok = false; break; }
          tc_fence_after();
          tmem_d = tmem_base + (uint32_t)(acc * BN);
        }
        if (!mbar_wait(smem_u32(&full_bar[s]), phase)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)     // 32 bytes further along K: +2 in units of 16 bytes
          umma_f16(tmem_d, desc_hi | (a_lo[s] + 2 * k), desc_hi | (b_lo[s] + 2 * k), idesc, (kb | k) ? 1u : 0u);
        umma_commit(smem_u32(&empty_bar[s]));
        if (++kb == k_blocks) {
          kb = 0;
          umma_commit(smem_u32(&acc_full[acc]));
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
      }
      phase ^= 1;
    }
    if (!ok) {
      fmx_set_status(status, FMX_WAIT_EXPIRED, 2, blockIdx.x);
      // products issued before the wait ran out may still be running: the tensor memory they
      // write is not freed under them.  A commit arrives when all of them are done.
      umma_commit(smem_u32(drain_bar));
      mbar_wait(smem_u32(drain_bar), 0);
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;                  // the 32 lanes of tensor memory this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    constexpr int OUT_COLS = EPI == EPI_SILU_MUL ? BN / 2 : BN;
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
      const int m0 = (t % tiles_m) * BM, n_tile = t / tiles_m;
      if (!mbar_wait(smem_u32(&acc_full[acc]), acc_phase)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
      const int out_n0 = n_tile * OUT_COLS;
      const int n_out = EPI == EPI_SILU_MUL ? N / 2 : N;
#pragma unroll 1
      for (int c = 0; c < OUT_COLS; c += 16) {
        uint32_t v[16], u[16];
        tmem_ld16(taddr + c, v);
        if (EPI == EPI_SILU_MUL) tmem_ld16(taddr + BN / 2 + c, u);
        tmem_ld_wait();
        if (row < M) {
          float f[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            f[i] = __uint_as_float(v[i]);
            if (EPI == EPI_SILU_MUL) {
              // as the unfused path rounds: gate and up to bfloat16 first, then the product
              const float g = __bfloat162float(__float2bfloat16_rn(f[i]));
              const float w = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[i])));
              f[i] = silu(g) * w;
            }
          }
          const int col = out_n0 + c;
          bf16* dst = C + (long long)row * ldc + col;
          if (EPI == EPI_RESIDUAL) {
            const bf16* rp = residual + (long long)row * ldr + col;
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (col + i < n_out) f[i] = __bfloat162float(__float2bfloat16_rn(f[i])) + __bfloat162float(rp[i]);
          }
          if (col + 16 <= n_out && (((uintptr_t)dst) & 15) == 0) {
            uint4 a, b;
            a.x = pack2(f[0], f[1]); a.y = pack2(f[2], f[3]); a.z = pack2(f[4], f[5]); a.w = pack2(f[6], f[7]);
            b.x = pack2(f[8], f[9]); b.y = pack2(f[10], f[11]); b.z = pack2(f[12], f[13]); b.w = pack2(f[14], f[15]);
            reinterpret_cast<uint4*>(dst)[0] = a;
            reinterpret_cast<uint4*>(dst)[1] = b;
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (col + i < n_out) dst[i] = __float2bfloat16_rn(f[i]);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&acc_empty[acc]));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (!ok && lane == 0) fmx_set_status(status, FMX_WAIT_EXPIRED, 3, blockIdx.x);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(cfg::TMEM_COLS) : "memory");
  }
}

template <int BN, int EPI>
int run(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc, const void* residual,
        long long ldr, int M, int N, int K, int sms, int* status, cudaStream_t stream) {
  using cfg = Cfg<BN>;
  CUtensorMap map_a, map_w;
  if (make_map_k128(&map_a, A, M, K, lda, BM) || make_map_k128(&map_w, W, N, K, ldw, BN)) return 1;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)cfg::SMEM);
    if (e != cudaSuccess) return fmx_fail("gemm_tcgen05: %zu bytes of shared memory refused: %s", cfg::SMEM,
                                          cudaGetErrorString(e));
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sms ? tiles : sms;
  cudaError_t e = fmx_launch(gemm_tcgen05_kernel<BN, EPI>, dim3(grid), dim3(THREADS), cfg::SMEM, stream, map_a, map_w,
                             (bf16*)C, ldc, (const bf16*)residual, ldr, M, N, K, status);
  if (e != cudaSuccess) return fmx_fail("gemm_tcgen05: launch failed: %s", cudaGetErrorString(e));
  return 0;
}
}  // namespace

// The tile width (of 128, 192, 256) whose tiles fill the SMs' rounds best; wider wins ties.
FMX_EXPORT int fmx_gemm_tcgen05_plan_width(int M, int N, int sms) {
  if (sms <= 0) sms = fmx_num_sms();
  int best = 256;
  double best_eff = -1.0;
  const int widths[3] = {256, 192, 128};
  for (int bn : widths) {
    const long long tiles = (long long)((M + 127) / 128) * ((N + bn - 1) / bn);
    const long long rounds = (tiles + sms - 1) / sms;
    const double eff = (double)tiles / (double)(rounds * sms) * ((double)N / (double)(((N + bn - 1) / bn) * bn)) *
                       (bn == 128 ? 0.8 : 1.0);
    if (eff > best_eff + 1e-9) { best = bn; best_eff = eff; }
  }
  return best;
}

// Does this product fill the GPU here?  The kernel gives each CTA whole tiles and walks K serially
// within a tile.  With fewer tiles than about a round of the SMs (short prompts against the
// narrower matrices) most SMs idle behind that walk, and the library's product, which splits K, is
// two to three times faster (512 x 2048 x 8192: 41 us against 17); with full rounds the two are
// within a tenth.  The same holds when the last round of tiles is mostly empty (192 tiles: two
// rounds for the work of 1.3; 2048 x 3072 x 2048 takes 28.9 us here against 19.8 in the library).
FMX_EXPORT int fmx_gemm_tcgen05_plan_fills(int M, int N, int sms) {
  if (sms <= 0) sms = fmx_num_sms();
  const long long tiles = (long long)((M + 127) / 128) * ((N + 255) / 256);
  const long long rounds = (tiles + sms - 1) / sms;
  return (double)tiles >= 0.8 * sms && (double)tiles >= 0.75 * (double)(rounds * sms) ? 1 : 0;
}

// A [M, K], W [N, K] bfloat16 with K-contiguous rows whose starts are 16-byte aligned; C
// bfloat16 [M, N] (EPI 0, 2) or [M, N/2] (EPI 1, W's rows in blocks of bn/2 gate rows then
// bn/2 up rows).  bn is 128, 192 (plain only) or 256, or 0 for the width that fills the SMs best
// (256 with the SiLU-mul epilogue).  status: the engine's status word (a wait that expires
// leaves FMX_WAIT_EXPIRED there).
FMX_EXPORT int fmx_gemm_tcgen05(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc,
                                const void* residual, long long ldr, int M, int N, int K, int bn, int epilogue,
                                int sms, int* status, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || N < 0 || K <= 0) return fmx_fail("fmx_gemm_tcgen05: bad sizes M=%d N=%d K=%d", M, N, K);
  if (K % 8 || lda % 8 || ldw % 8 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15))
    return fmx_fail("fmx_gemm_tcgen05: rows must start on 16-byte boundaries (K=%d lda=%lld ldw=%lld)", K, lda, ldw);
  if (bn == 0) bn = epilogue == EPI_SILU_MUL ? 256 : fmx_gemm_tcgen05_plan_width(M, N, sms);
  if (epilogue == EPI_SILU_MUL && N % bn) return fmx_fail("fmx_gemm_tcgen05: gate/up blocks need N a multiple of %d", bn);
  if (epilogue == EPI_RESIDUAL && residual == nullptr) return fmx_fail("fmx_gemm_tcgen05: the residual epilogue needs a residual");
  if (sms <= 0) sms = fmx_num_sms();
#define FMX_TC_CASE(BN_, EPI_) \
  if (bn == BN_ && epilogue == EPI_) return run<BN_, EPI_>(A, lda, W, ldw, C, ldc, residual, ldr, M, N, K, sms, status, stream)
  FMX_TC_CASE(256, EPI_PLAIN);
  FMX_TC_CASE(192, EPI_PLAIN);
  FMX_TC_CASE(128, EPI_PLAIN);
  FMX_TC_CASE(256, EPI_SILU_MUL);
  FMX_TC_CASE(128, EPI_SILU_MUL);
  FMX_TC_CASE(256, EPI_RESIDUAL);
  FMX_TC_CASE(128, EPI_RESIDUAL);
#undef FMX_TC_CASE
  return fmx_fail("fmx_gemm_tcgen05: no kernel for tile width %d, epilogue %d", bn, epilogue);
}
