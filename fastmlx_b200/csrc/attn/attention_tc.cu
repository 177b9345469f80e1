// Paged causal attention for prompt portions on the fifth-generation tensor cores
// (head sizes 64 and 128; compile with -DFMX_HD=<head size>).
//
// Query rows are "packed": row i of a tile stands for token i / rep and query head
// g*rep + i % rep (rep = query heads per kv head), so that all rows of a tile read the same
// keys and values; a tile holds 128 / rep tokens (its last rows are idle when rep does not
// divide 128).  Two kernels:
//
//  * two query tiles per CTA (the default; further down, namespace `two`): tiles A and B share
//    every K/V tile, each with its own softmax group of four warps and one thread per row;
//  * one query tile per CTA (below): eight softmax warps, two threads per row.  It remains
//    for page sizes that do not divide the other kernel's key tile.
//
// The one-tile kernel: a CTA owns 128 packed query rows of one request and one kv head and
// walks over the keys in tiles of 128.
//   warp 0           : producer.  One 3-D TMA load brings the query tile; per key tile, one
//                      2-D TMA load per page (one lane per page, so that the block-table reads
//                      of a tile overlap) brings K and one brings V (a page of a kv head is a
//                      contiguous [page_size, hd] block of the cache), all with the 128-byte
//                      swizzle the MMA expects.  Pages beyond the last visible key are replaced
//                      by an out-of-bounds box, which TMA fills with zeros.
//   warp 1, one lane : MMA issuer.  S_j = Q K_j^T (tcgen05.mma, both operands K-major) into one
//                      of two score buffers in tensor memory, then, one tile behind, O_j = P_j V_j
//                      (P from shared memory, V as an MN-major operand) into one of two output
//                      buffers: the tensor core computes S_{j+1} while the softmax of tile j runs.
//   warps 2-9        : softmax and epilogue, two threads per query row (64 keys and half of the
//                      head dimension each; the halves' maxima meet through shared memory).
//                      Scores come from tensor memory (tcgen05.ld), running maximum and sum are
//                      32-bit, probabilities go to shared memory in bfloat16, the per-tile outputs
//                      are rescaled and summed in registers.
// Every barrier wait is bounded by time; a wait that runs out leaves FMX_WAIT_EXPIRED in the
// status word and the CTA frees its tensor memory and returns.  No cluster: every CTA loads its own tiles.
#include <cuda.h>
#include <math.h>
#include <type_traits>
#include "common.cuh"
#include "tcgen05.cuh"

#ifndef FMX_HD
#error "compile with -DFMX_HD=<head size>"
#endif

#if FMX_HD == 64 || FMX_HD == 128
namespace {
using namespace fmx_tc;
constexpr int HD = FMX_HD;
constexpr int KB = HD / 64;                    // 64-wide blocks of the head dimension
constexpr int BM = 128, BN = 128;
constexpr int TILE_BYTES = 128 * 128;          // a [128 x 64] bfloat16 block, 128-byte rows
constexpr int KV_STAGES = HD == 64 ? 3 : 2;
constexpr int P_BUFS = HD == 64 ? 2 : 1;
constexpr int Q_BYTES = KB * TILE_BYTES, K_BYTES = KB * TILE_BYTES, V_BYTES = KB * TILE_BYTES;
constexpr int P_BYTES = 2 * TILE_BYTES;        // 128 rows x 128 keys
constexpr int THREADS = 320;                  // producer, MMA issuer, eight softmax warps
constexpr int SOFTMAX_THREADS = 256;
constexpr int TMEM_COLS = 512;
constexpr int S_COL = 0, O_COL = 256;          // S0, S1 at 0, 128; O0, O1 at 256, 256 + HD
constexpr float LOG2E = 1.4426950408889634f;
constexpr size_t SMEM_BYTES = (size_t)Q_BYTES + (size_t)KV_STAGES * (K_BYTES + V_BYTES) + (size_t)P_BUFS * P_BYTES +
                              1024 + 512 + 2 * 2 * 128 * 4;

// 2^x by the special-function unit (about two units in the last place; -inf gives 0).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

struct Bars {
  uint64_t q_full;
  uint64_t kv_full[KV_STAGES], kv_empty[KV_STAGES];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full[P_BUFS], p_empty[P_BUFS];
  uint64_t o_full[2], o_empty[2];
  uint64_t x_bar[2];                           // the two column halves meet here (256 arrivals)
  uint32_t tmem_slot;
  float xmax[2][2][128];                       // [tile parity][column half][row]: the halves' maxima
};

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                       const int* block_tables, int bt_stride, const int* row_start, const int* row_ctx, bf16* out,
                       int nh, int nkv, int page_size, long long num_pages, long long kv_rows, float scale,
                       int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sq = smem;
  unsigned char* skv = sq + Q_BYTES;                                   // [stage][K | V]
  unsigned char* sp = skv + (size_t)KV_STAGES * (K_BYTES + V_BYTES);   // [P_BUFS]
  Bars* bars = reinterpret_cast<Bars*>(sp + (size_t)P_BUFS * P_BYTES);

  // The last query tiles of a row see the most keys.  Blocks start in the order x, y, z: with the
  // tile index in z the longest blocks of every head and row start first and the short ones fill in
  // behind them (with it in x, the last heads' long blocks started late and ran on alone).
  const int r = blockIdx.y, g = blockIdx.x, tile = gridDim.z - 1 - blockIdx.z;
  const int rep = nh / nkv;
  const int tok_per_tile = BM / rep;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bars->q_full), 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(smem_u32(&bars->kv_full[s]), 1);
      mbar_init(smem_u32(&bars->kv_empty[s]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars->s_full[i]), 1);
      mbar_init(smem_u32(&bars->s_empty[i]), SOFTMAX_THREADS);
      mbar_init(smem_u32(&bars->o_full[i]), 1);
      mbar_init(smem_u32(&bars->o_empty[i]), SOFTMAX_THREADS);
    }
    for (int i = 0; i < 2; ++i) mbar_init(smem_u32(&bars->x_bar[i]), SOFTMAX_THREADS);
    for (int i = 0; i < P_BUFS; ++i) {
      mbar_init(smem_u32(&bars->p_full[i]), SOFTMAX_THREADS);
      mbar_init(smem_u32(&bars->p_empty[i]), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_slot;
  pdl_wait();
  pdl_trigger();

  const int t0 = row_start[r], q_len = row_start[r + 1] - t0, ctx = row_ctx[r];
  const int tok0 = tile * tok_per_tile;                   // first token of this tile within the row
  const bool active = tok0 < q_len && ctx >= 0;
  const int n_tok = active ? min(tok_per_tile, q_len - tok0) : 0;
  const int kend = ctx + tok0 + n_tok;                    // one past the last key any row of the tile sees
  const int n_tiles = active ? (kend + BN - 1) / BN : 0;
  const int pages_per_tile = BN / page_size;

  if (warp == 0 && active) {
    // ------------------------------------------------------------------ producer
    // The whole warp: lane 0 owns the barriers; lane p looks up page p of the tile and issues
    // its copies, so that the block-table reads of a tile overlap instead of queueing.
    const int* bt = block_tables + (long long)r * bt_stride;
    if (lane == 0) {
      // the box holds tok_per_tile x rep rows: all 128 when rep divides 128, else the last few
      // rows of the tile are left as they are (they belong to no token and are never stored)
      mbar_expect_tx(smem_u32(&bars->q_full), (uint32_t)(tok_per_tile * rep * 128 * KB));
#pragma unroll
      for (int kb = 0; kb < KB; ++kb)
        tma_load_3d(smem_u32(sq + kb * TILE_BYTES), &map_q, kb * 64, g * rep, t0 + tok0, smem_u32(&bars->q_full));
    }
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const uint32_t fb = smem_u32(&bars->kv_full[stage]);
      if (lane == 0) {
        ok = mbar_wait(smem_u32(&bars->kv_empty[stage]), phase ^ 1);
        if (ok) mbar_expect_tx(fb, K_BYTES + V_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (lane < pages_per_tile) {
        const int pi = lane;
        unsigned char* sk = skv + (size_t)stage * (K_BYTES + V_BYTES);
        unsigned char* sv = sk + K_BYTES;
        const int key0 = j * BN + pi * page_size;
        long long krow = kv_rows, vrow = kv_rows;           // out of bounds: the box reads as zeros
        if (key0 < kend) {
          const int blk = key0 / page_size;
          const int page = blk < bt_stride ? bt[blk] : -1;
          if (page < 0 || page >= num_pages) {
            fmx_set_status(status, FMX_BAD_PAGE, page, r);
          } else {
            krow = (((long long)page * 2 + 0) * nkv + g) * page_size;
            vrow = (((long long)page * 2 + 1) * nkv + g) * page_size;
          }
        }
        const int off = pi * page_size * 128;               // rows of 128 bytes
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
          tma_load_2d(smem_u32(sk + kb * TILE_BYTES + off), &map_kv, kb * 64, (int)krow, fb);
          tma_load_2d(smem_u32(sv + kb * TILE_BYTES + off), &map_kv, kb * 64, (int)vrow, fb);
        }
      }
      if (++stage == KV_STAGES) { stage = 0; phase ^= 1; }
    }
    if (!ok && lane == 0) fmx_set_status(status, FMX_WAIT_EXPIRED, 11, blockIdx.x);
  } else if (warp == 1 && lane == 0 && active) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc_qk = make_idesc(BM, BN, 0), idesc_pv = make_idesc(BM, HD, 1);
    bool ok = mbar_wait(smem_u32(&bars->q_full), 0);
    tc_fence_after();
    auto issue_pv = [&](int j) -> bool {
      const int st = j % KV_STAGES, pb = j % P_BUFS, ob = j & 1;
      if (!mbar_wait(smem_u32(&bars->p_full[pb]), (uint32_t)((j / P_BUFS) & 1))) return false;
      if (!mbar_wait(smem_u32(&bars->o_empty[ob]), (uint32_t)(((j >> 1) & 1) ^ 1))) return false;
      tc_fence_after();
      const uint32_t pa = smem_u32(sp + (size_t)pb * P_BYTES);
      const uint32_t va = smem_u32(skv + (size_t)st * (K_BYTES + V_BYTES) + K_BYTES);
#pragma unroll
      for (int kb = 0; kb < 2; ++kb)          // 64 keys each
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)        // 16 keys each
          umma_f16(tmem + O_COL + ob * HD, make_desc_k128(pa + kb * TILE_BYTES) + 2 * k4,
               make_desc_mn128(va + (kb * 64 + k4 * 16) * 128, TILE_BYTES), idesc_pv, (kb | k4) ? 1u : 0u);
      umma_commit(smem_u32(&bars->o_full[ob]));
      umma_commit(smem_u32(&bars->p_empty[pb]));
      umma_commit(smem_u32(&bars->kv_empty[st]));
      return true;
    };
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j % KV_STAGES, sb = j & 1;
      if (!mbar_wait(smem_u32(&bars->kv_full[st]), (uint32_t)((j / KV_STAGES) & 1))) { ok = false; break; }
      if (!mbar_wait(smem_u32(&bars->s_empty[sb]), (uint32_t)(((j >> 1) & 1) ^ 1))) { ok = false; break; }
      tc_fence_after();
      const uint32_t qa = smem_u32(sq), ka = smem_u32(skv + (size_t)st * (K_BYTES + V_BYTES));
#pragma unroll
      for (int kb = 0; kb < KB; ++kb)
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
          umma_f16(tmem + S_COL + sb * BN, make_desc_k128(qa + kb * TILE_BYTES) + 2 * k4,
               make_desc_k128(ka + kb * TILE_BYTES) + 2 * k4, idesc_qk, (kb | k4) ? 1u : 0u);
      umma_commit(smem_u32(&bars->s_full[sb]));
      if (j > 0) ok = issue_pv(j - 1);
    }
    if (ok && n_tiles > 0) ok = issue_pv(n_tiles - 1);
    if (!ok) fmx_set_status(status, FMX_WAIT_EXPIRED, 12, blockIdx.x);
  } else if (warp >= 2 && active) {
    // ------------------------------------------------------------------ softmax and epilogue
    // Two threads per query row: warps 2-5 take the first 64 keys of every tile and the first
    // half of the head dimension of the output, warps 6-9 the second halves.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;                 // this thread's packed row and tensor-memory lane
    const int tok = row / rep, head = g * rep + row - tok * rep;
    const bool rvalid = tok < n_tok;
    const int lim = rvalid ? ctx + tok0 + tok : -1;      // last key this row sees
    const float sl2 = scale * LOG2E;
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    constexpr int OH = HD / 2;                           // output columns of this thread
    float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
    float o[OH];
#pragma unroll
    for (int d = 0; d < OH; ++d) o[d] = 0.f;
    bool ok = true;

    auto take_output = [&](int j, float alpha) -> bool {   // o = o * alpha + (P_j V_j)[row, this half]
      const int ob = j & 1;
      if (!mbar_wait(smem_u32(&bars->o_full[ob]), (uint32_t)((j >> 1) & 1))) return false;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < OH; c += 32) {
        uint32_t v[32];
        tmem_ld32(lane_addr + O_COL + ob * HD + half * OH + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c + i] = fmaf(o[c + i], alpha, __uint_as_float(v[i]));
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&bars->o_empty[ob]));
      return true;
    };

    for (int j = 0; j < n_tiles && ok; ++j) {
      const int sb = j & 1, pb = j % P_BUFS, st = j % KV_STAGES;
      if (!mbar_wait(smem_u32(&bars->s_full[sb]), (uint32_t)((j >> 1) & 1))) { ok = false; break; }
      tc_fence_after();
      const int key0 = j * BN + half * 64;               // first key of this thread's 64 columns
      const bool need_mask = j * BN + BN - 1 > ctx + tok0;  // some row of the tile does not see the whole tile
      uint32_t v0[32], v1[32];
      tmem_ld32(lane_addr + S_COL + sb * BN + half * 64, v0);
      tmem_ld32(lane_addr + S_COL + sb * BN + half * 64 + 32, v1);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(smem_u32(&bars->s_empty[sb]));         // the scores are in registers now
      float sc[64];
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        sc[i] = (!need_mask || key0 + i <= lim) ? __uint_as_float(v0[i]) * sl2 : -INFINITY;
        sc[32 + i] = (!need_mask || key0 + 32 + i <= lim) ? __uint_as_float(v1[i]) * sl2 : -INFINITY;
        mx = fmaxf(mx, fmaxf(sc[i], sc[32 + i]));
      }
      // the row's maximum over the whole tile: exchange with the thread that has the other half
      bars->xmax[j & 1][half][row] = mx;
      mbar_arrive(smem_u32(&bars->x_bar[j & 1]));
      if (!mbar_wait(smem_u32(&bars->x_bar[j & 1]), (uint32_t)((j >> 1) & 1))) { ok = false; break; }
      mx = fmaxf(mx, bars->xmax[j & 1][half ^ 1][row]);
      const float m_new = fmaxf(m, mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = fast_exp2(m - m_use);
      m = m_new;
      if (!mbar_wait(smem_u32(&bars->p_empty[pb]), (uint32_t)(((j / P_BUFS) & 1) ^ 1))) { ok = false; break; }
      // probabilities to shared memory (K-major, 128-byte rows, swizzled by row): this thread's
      // 64 keys are the k block `half` of the tile
      unsigned char* prow = sp + (size_t)pb * P_BYTES + half * TILE_BYTES + row * 128;
      float sum = 0.f;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        float pr[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          pr[i] = fast_exp2(sc[8 * ch + i] - m_use);
          sum += pr[i];
        }
        uint4 w;
        w.x = pack2(pr[0], pr[1]);
        w.y = pack2(pr[2], pr[3]);
        w.z = pack2(pr[4], pr[5]);
        w.w = pack2(pr[6], pr[7]);
        *reinterpret_cast<uint4*>(prow + ((ch ^ (row & 7)) << 4)) = w;
      }
      l = l * alpha + sum;
      if (j * BN + BN > kend && half == 0) {
        // keys past the last visible one share pages with stale rows: their values must be
        // zeros, since 0 * NaN would poison the product
        if (!mbar_wait(smem_u32(&bars->kv_full[st]), (uint32_t)((j / KV_STAGES) & 1))) { ok = false; break; }
        unsigned char* sv = skv + (size_t)st * (K_BYTES + V_BYTES) + K_BYTES;
        if (j * BN + row >= kend) {
#pragma unroll
          for (int kb = 0; kb < KB; ++kb)
#pragma unroll
            for (int ch = 0; ch < 8; ++ch)
              *reinterpret_cast<uint4*>(sv + kb * TILE_BYTES + row * 128 + ch * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(smem_u32(&bars->p_full[pb]));
      // one tile behind: add the previous tile's output
      if (j > 0) ok = take_output(j - 1, alpha_prev);
      alpha_prev = alpha;
    }
    if (ok && n_tiles > 0) ok = take_output(n_tiles - 1, alpha_prev);
    // the row's sum: both halves saw the same maxima, so their sums just add
    if (ok) {
      // tile n_tiles uses the exchange buffers of that parity: nobody reads them any more
      const int jx = n_tiles;
      bars->xmax[jx & 1][half][row] = l;
      mbar_arrive(smem_u32(&bars->x_bar[jx & 1]));
      ok = mbar_wait(smem_u32(&bars->x_bar[jx & 1]), (uint32_t)((jx >> 1) & 1));
      l += bars->xmax[jx & 1][half ^ 1][row];
    }
    if (!ok) {
      if (lane == 0) fmx_set_status(status, FMX_WAIT_EXPIRED, 13, blockIdx.x);
    } else if (rvalid) {
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      bf16* op = out + ((long long)(t0 + tok0 + tok) * nh + head) * HD + half * OH;
#pragma unroll
      for (int c = 0; c < OH; c += 8) {
        uint4 w;
        w.x = pack2(o[c] * inv, o[c + 1] * inv);
        w.y = pack2(o[c + 2] * inv, o[c + 3] * inv);
        w.z = pack2(o[c + 4] * inv, o[c + 5] * inv);
        w.w = pack2(o[c + 6] * inv, o[c + 7] * inv);
        *reinterpret_cast<uint4*>(op + c) = w;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------
// Two query tiles per CTA.  The CTA owns 256 packed query rows: tile A (rows
// 0-127) and tile B (rows 128-255) share every K/V tile that TMA brings, and each has a
// softmax group of four warps with one thread per query row, so no row statistic ever
// crosses a thread.  While one group works on its scores the tensor core computes the other
// tile's, and K and V are read from shared memory once for 256 rows.
// Head size 64: keys in tiles of 128; tensor memory holds S_A, S_B (one column per key), O_A, O_B
// (one per head dimension) and P_A, P_B (the probabilities in bfloat16, two keys per column), 512
// columns; shared memory Q_A, Q_B and four K/V stages of 32 KB.  A softmax thread reads its row
// of scores twice, 64 columns at a time (once for the maximum, once for the exponentials); the
// next Q K^T of its query tile starts when it has.
// Head size 128: scores and outputs alone would fill tensor memory at 128 keys a tile, so keys come
// in tiles of 64 and every query tile has two score buffers: the Q K^T of tile j + 1 runs while
// the softmax works on tile j.  A row of 64 scores is taken into registers at once; the
// probabilities are written over the first half of the tile's own scores, which stay held until
// the P V product has read them.  Two threads issue the products there, one the scores and one
// P V: with one, a product whose inputs were ready waited behind the other three kinds, since an
// issue call lasts as long as the tensor pipe is busy (8 x 256 tokens over 4,096 cached: 228 us
// with one score buffer, 214 with two, 179 with two issuers as well; the same two changes at head
// size 64 lose to its 128-key tiles, 144 against 134 us).
// In both, the P V product reads P from tensor memory (A operand) and V from shared memory, and the
// outputs stay in tensor memory: every P V product accumulates onto them, and a row's
// output is rescaled there only when its running maximum has grown by more than 2^8 since the
// scale in use was fixed (probabilities then stay below 2^8, far inside bfloat16 and 32-bit
// range; the final division by the row sum, kept at the same scale, undoes it exactly).
namespace two {
// DB: two score buffers per query tile and two issuing threads (head size 128, see above).
#ifndef FMX_ATTN_DB
#define FMX_ATTN_DB (FMX_HD == 128)
#endif
constexpr bool DB = FMX_ATTN_DB;
constexpr int BN2 = DB ? 64 : (HD == 64 ? 128 : 64);   // keys per tile
constexpr int KV_ST = 4;
constexpr int K2_BYTES = KB * BN2 * 128, V2_BYTES = K2_BYTES;      // KB blocks of [BN2 keys][64 dims]
constexpr int THREADS2 = DB ? 352 : 320;        // producer, MMA issuer, 4 + 4 softmax warps; DB: a second issuer
constexpr int GROUP_THREADS = 128;
constexpr size_t SMEM2 = 2 * (size_t)Q_BYTES + (size_t)KV_ST * (K2_BYTES + V2_BYTES) + 1024 + 512;
constexpr int S2_COL = 0, O2_COL = DB ? 4 * BN2 : 2 * BN2, P2_COL = O2_COL + 2 * HD;   // P: two keys per column
static_assert((DB ? O2_COL + 2 * HD : P2_COL + BN2) <= TMEM_COLS, "scores, outputs and probabilities must fit tensor memory");

struct Bars2 {
  uint64_t q_full;
  uint64_t kv_full[KV_ST], kv_empty[KV_ST];
  uint64_t s_full[2], s_empty[2];               // per query tile
  uint64_t p_full[2], p_empty[2];
  uint64_t o_full[2];                           // per query tile: a P V product has landed
  uint64_t sd_full[2][2], pd_full[2][2], pv_done[2][2];   // DB: per query tile and score buffer
  uint32_t tmem_slot;
};

__global__ void __launch_bounds__(THREADS2, 1)
attn_prefill_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                        const int* block_tables, int bt_stride, const int* row_start, const int* row_ctx, bf16* out,
                        int nh, int nkv, int page_size, long long num_pages, long long kv_rows, float scale,
                        int* status, int ksplits, float* part_o, float* part_ml, int T) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sq = smem;                                             // [2] query tiles
  unsigned char* skv = sq + 2 * Q_BYTES;                                // [stage][K | V]
  Bars2* bars = reinterpret_cast<Bars2*>(skv + (size_t)KV_ST * (K2_BYTES + V2_BYTES));

  // the pairs that see the most keys start first, for every head and row (see the one-tile kernel)
  // With `ksplits` > 1 the keys of a pair of query tiles are shared out over that many CTAs (z = pair * ksplits +
  // split): each leaves unnormalised outputs with their scale and sum, and a second kernel combines them.  That is
  // for grids that would leave most SMs idle: one 512-token portion behind tens of thousands of keys.
  const int r = blockIdx.y, g = blockIdx.x, zz = gridDim.z - 1 - blockIdx.z;
  const int pair = zz / ksplits, split = zz - pair * ksplits;
  const int rep = nh / nkv;
  const int tok_per_tile = BM / rep;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bars->q_full), 1);
    for (int s = 0; s < KV_ST; ++s) {
      mbar_init(smem_u32(&bars->kv_full[s]), 1);
      mbar_init(smem_u32(&bars->kv_empty[s]), 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(smem_u32(&bars->s_full[x]), 1);
      mbar_init(smem_u32(&bars->s_empty[x]), GROUP_THREADS);
      mbar_init(smem_u32(&bars->p_full[x]), GROUP_THREADS);
      mbar_init(smem_u32(&bars->p_empty[x]), 1);
      mbar_init(smem_u32(&bars->o_full[x]), 1);
      for (int b = 0; b < 2; ++b) {
        mbar_init(smem_u32(&bars->sd_full[x][b]), 1);
        mbar_init(smem_u32(&bars->pd_full[x][b]), GROUP_THREADS);
        mbar_init(smem_u32(&bars->pv_done[x][b]), 1);
      }
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_slot;
  pdl_wait();
  pdl_trigger();

  const int t0 = row_start[r], q_len = row_start[r + 1] - t0, ctx = row_ctx[r];
  // per query tile: first token, tokens, one past the last key any of its rows sees, key tiles
  const int tok0_a = 2 * pair * tok_per_tile, tok0_b = tok0_a + tok_per_tile;
  const bool act_a = tok0_a < q_len && ctx >= 0, act_b = tok0_b < q_len && ctx >= 0;
  const int n_tok_a = act_a ? min(tok_per_tile, q_len - tok0_a) : 0, n_tok_b = act_b ? min(tok_per_tile, q_len - tok0_b) : 0;
  const int kend_a = ctx + tok0_a + n_tok_a, kend_b = ctx + tok0_b + n_tok_b;
  const int all_a = act_a ? (kend_a + BN2 - 1) / BN2 : 0, all_b = act_b ? (kend_b + BN2 - 1) / BN2 : 0;
  // this CTA's key tiles: [j0, j0 + per) of the pair's; below, j counts from j0 and a tile's first key is (j0 + j) BN2
  const int per = (max(all_a, all_b) + ksplits - 1) / ksplits, j0 = split * per;
  const int n_tiles_a = min(max(all_a - j0, 0), per), n_tiles_b = min(max(all_b - j0, 0), per);
  const int n_all = max(n_tiles_a, n_tiles_b);         // tile B sees at least what A sees
  const int kend_all = max(act_a ? kend_a : 0, act_b ? kend_b : 0);
  const int pages_per_tile = BN2 / page_size;

  if (warp == 0 && n_all > 0) {
    // ------------------------------------------------------------------ producer
    // The whole warp: lane 0 owns the barriers; lane p looks up page p of the tile and issues
    // its two copies, so that the block-table reads of a tile overlap instead of queueing.
    const int* bt = block_tables + (long long)r * bt_stride;
    if (lane == 0) {
      // a box holds tok_per_tile x rep rows: all 128 when rep divides 128, else the last few
      // rows of a tile are left as they are (they belong to no token and are never stored)
      mbar_expect_tx(smem_u32(&bars->q_full), (uint32_t)(2 * tok_per_tile * rep * 128 * KB));
#pragma unroll
      for (int x = 0; x < 2; ++x)             // a tile past the row's end reads as zeros
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_3d(smem_u32(sq + x * Q_BYTES + kb * TILE_BYTES), &map_q, kb * 64, g * rep, t0 + (x ? tok0_b : tok0_a),
                      smem_u32(&bars->q_full));
    }
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int j = 0; j < n_all; ++j) {
      const uint32_t fb = smem_u32(&bars->kv_full[stage]);
      if (lane == 0) {
        ok = mbar_wait(smem_u32(&bars->kv_empty[stage]), phase ^ 1);
        if (ok) mbar_expect_tx(fb, K2_BYTES + V2_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (lane < pages_per_tile) {
        const int pi = lane;
        unsigned char* sk = skv + (size_t)stage * (K2_BYTES + V2_BYTES);
        unsigned char* sv = sk + K2_BYTES;
        const int key0 = (j0 + j) * BN2 + pi * page_size;
        long long krow = kv_rows, vrow = kv_rows;           // out of bounds: the box reads as zeros
        if (key0 < kend_all) {
          const int blk = key0 / page_size;
          const int page = blk < bt_stride ? bt[blk] : -1;
          if (page < 0 || page >= num_pages) {
            fmx_set_status(status, FMX_BAD_PAGE, page, r);
          } else {
            krow = (((long long)page * 2 + 0) * nkv + g) * page_size;
            vrow = (((long long)page * 2 + 1) * nkv + g) * page_size;
          }
        }
        const int off = pi * page_size * 128;               // rows of 128 bytes
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
          tma_load_2d(smem_u32(sk + kb * BN2 * 128 + off), &map_kv, kb * 64, (int)krow, fb);
          tma_load_2d(smem_u32(sv + kb * BN2 * 128 + off), &map_kv, kb * 64, (int)vrow, fb);
        }
      }
      if (++stage == KV_ST) { stage = 0; phase ^= 1; }
    }
    if (!ok && lane == 0) fmx_set_status(status, FMX_WAIT_EXPIRED, 21, blockIdx.x);
  } else if ((warp == 1 || (DB && warp == 10)) && lane == 0 && n_all > 0) {
    // ------------------------------------------------------------------ MMA issuer(s)
    const uint32_t idesc_qk = make_idesc(BM, BN2, 0), idesc_pv = make_idesc(BM, HD, 1);
    bool ok = mbar_wait(smem_u32(&bars->q_full), 0);
    tc_fence_after();
    // The two query tiles advance independently: whichever product has its inputs goes next
    // (scores of tile j need its K tile and the score buffer read out; P V of tile j needs its
    // probabilities), so one tile's softmax never waits for the other's.
    auto issue_qk = [&](int x, int j) {
      const int st = j % KV_ST;
      const uint32_t q_lo = desc_lo_k128(smem_u32(sq + x * Q_BYTES));
      const uint32_t k_lo = desc_lo_k128(smem_u32(skv + (size_t)st * (K2_BYTES + V2_BYTES)));
#pragma unroll
      for (int kb = 0; kb < KB; ++kb)
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
          umma_f16(tmem + S2_COL + x * BN2, desc_sw128(q_lo + (kb * TILE_BYTES >> 4) + 2 * k4),
                   desc_sw128(k_lo + (kb * BN2 * 128 >> 4) + 2 * k4), idesc_qk, (kb | k4) ? 1u : 0u);
      umma_commit(smem_u32(&bars->s_full[x]));
    };
    auto issue_pv = [&](int x, int j) {
      const int st = j % KV_ST;
      const uint32_t pa = tmem + P2_COL + x * (BN2 / 2);
      const uint32_t v_lo = desc_lo_mn128(smem_u32(skv + (size_t)st * (K2_BYTES + V2_BYTES) + K2_BYTES), BN2 * 128);
#pragma unroll
      for (int k = 0; k < BN2 / 16; ++k)      // 16 keys each; the first tile's first MMA starts the sum
        umma_f16_ts(tmem + O2_COL + x * HD, pa + 8 * k, desc_sw128(v_lo + (k * 16 * 128 >> 4)), idesc_pv,
                    (j > 0 || k) ? 1u : 0u);
      umma_commit(smem_u32(&bars->o_full[x]));
      umma_commit(smem_u32(&bars->p_empty[x]));
    };
    // DB: tile j of query tile x uses score buffer j & 1 for the (j >> 1)-th time; the buffer is
    // free again when the P V product of tile j - 2 has read its probabilities out of it.
    auto issue_qk_db = [&](int x, int j) {
      const int st = j % KV_ST;
      const uint32_t q_lo = desc_lo_k128(smem_u32(sq + x * Q_BYTES));
      const uint32_t k_lo = desc_lo_k128(smem_u32(skv + (size_t)st * (K2_BYTES + V2_BYTES)));
#pragma unroll
      for (int kb = 0; kb < KB; ++kb)
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
          umma_f16(tmem + S2_COL + (2 * x + (j & 1)) * BN2, desc_sw128(q_lo + (kb * TILE_BYTES >> 4) + 2 * k4),
                   desc_sw128(k_lo + (kb * BN2 * 128 >> 4) + 2 * k4), idesc_qk, (kb | k4) ? 1u : 0u);
      umma_commit(smem_u32(&bars->sd_full[x][j & 1]));
    };
    auto issue_pv_db = [&](int x, int j) {
      const int st = j % KV_ST;
      const uint32_t pa = tmem + S2_COL + (2 * x + (j & 1)) * BN2;
      const uint32_t v_lo = desc_lo_mn128(smem_u32(skv + (size_t)st * (K2_BYTES + V2_BYTES) + K2_BYTES), BN2 * 128);
#pragma unroll
      for (int k = 0; k < BN2 / 16; ++k)
        umma_f16_ts(tmem + O2_COL + x * HD, pa + 8 * k, desc_sw128(v_lo + (k * 16 * 128 >> 4)), idesc_pv,
                    (j > 0 || k) ? 1u : 0u);
      umma_commit(smem_u32(&bars->pv_done[x][j & 1]));
    };
    int qk_a = 0, qk_b = 0, pv_a = 0, pv_b = 0, released = 0;
    long long t_last = clock64();
    while (ok && (DB && warp == 1 ? (qk_a < n_tiles_a || qk_b < n_tiles_b) : (pv_a < n_tiles_a || pv_b < n_tiles_b))) {
      bool progress = false;
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        int& qk = x ? qk_b : qk_a;
        int& pv = x ? pv_b : pv_a;
        const int n = x ? n_tiles_b : n_tiles_a;
        if constexpr (DB) {
          // Two issuers, warp 1 for the scores and warp 10 for the P V products, each counting only
          // its own: with one, a product that was ready waited behind the three other kinds (every
          // issue call lasts as long as the tensor pipe is busy), and the softmax for its scores.
          if (warp == 1 && qk < n && mbar_test(smem_u32(&bars->kv_full[qk % KV_ST]), (uint32_t)((qk / KV_ST) & 1)) &&
              mbar_test(smem_u32(&bars->pv_done[x][qk & 1]), (uint32_t)(((qk >> 1) & 1) ^ 1))) {
            tc_fence_after();
            issue_qk_db(x, qk);
            ++qk;
            progress = true;
          }
          if (warp != 1 && pv < n && mbar_test(smem_u32(&bars->pd_full[x][pv & 1]), (uint32_t)((pv >> 1) & 1))) {
            tc_fence_after();
            issue_pv_db(x, pv);
            ++pv;
            progress = true;
          }
          continue;
        }
        if (qk < n && mbar_test(smem_u32(&bars->kv_full[qk % KV_ST]), (uint32_t)((qk / KV_ST) & 1)) &&
            mbar_test(smem_u32(&bars->s_empty[x]), (uint32_t)((qk & 1) ^ 1))) {
          tc_fence_after();
          issue_qk(x, qk);
          ++qk;
          progress = true;
        }
        if (pv < qk && mbar_test(smem_u32(&bars->p_full[x]), (uint32_t)(pv & 1))) {
          tc_fence_after();
          issue_pv(x, pv);
          ++pv;
          progress = true;
        }
      }
      // a K/V stage goes back once both tiles' products over it have been issued
      while (!(DB && warp == 1) && released < n_all && (released >= n_tiles_a || pv_a > released) &&
             (released >= n_tiles_b || pv_b > released)) {
        umma_commit(smem_u32(&bars->kv_empty[released % KV_ST]));
        ++released;
      }
      if (progress) t_last = clock64();
      else if (clock64() - t_last > WAIT_CYCLES) ok = false;
    }
    if (!ok) fmx_set_status(status, FMX_WAIT_EXPIRED, warp == 1 ? 22 : 24, blockIdx.x);
  } else if (warp >= 2 && warp < 10) {
    // ------------------------------------------------------------------ softmax and epilogue
    const int x = (warp - 2) >> 2;                       // query tile of this group
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                 // this thread's packed row and tensor-memory lane
    const int tok = row / rep, head = g * rep + row - tok * rep;
    const int tok0 = x ? tok0_b : tok0_a, n_tok = x ? n_tok_b : n_tok_a;
    const bool rvalid = tok < n_tok;
    const int lim = rvalid ? ctx + tok0 + tok : -1;      // last key this row sees
    const float sl2 = scale * LOG2E;
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + S2_COL + x * BN2;
    const uint32_t o_addr = lane_addr + O2_COL + x * HD;
    const uint32_t p_addr = lane_addr + P2_COL + x * (BN2 / 2);
    // m: the scale in use (log2 domain), fixed until the running maximum outgrows it by 2^8
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    const int nt = x ? n_tiles_b : n_tiles_a;

    // the output so far is at the old scale: bring this warp's rows to the new one
    auto rescale_output = [&](float alpha) {
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        uint32_t v[32];
        tmem_ld32(o_addr + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
        tmem_st32(o_addr + c, v);
      }
      tmem_st_wait();
    };
    // keys past the last visible one share pages with stale rows: their values must be
    // zeros, since 0 * NaN would poison the product (both groups write the same zeros)
    auto zero_stale_values = [&](int j, int key0) -> bool {
      const int st = j % KV_ST;
      if (!mbar_wait(smem_u32(&bars->kv_full[st]), (uint32_t)((j / KV_ST) & 1))) return false;
      unsigned char* sv = skv + (size_t)st * (K2_BYTES + V2_BYTES) + K2_BYTES;
      if (row < BN2 && key0 + row >= kend_all) {
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(sv + kb * BN2 * 128 + row * 128 + ch * 16) = make_uint4(0u, 0u, 0u, 0u);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      return true;
    };

    if constexpr (DB) {
      static_assert(!DB || BN2 == 64, "a row of scores is taken into 64 registers");
      for (int j = 0; j < nt && ok; ++j) {
        const int b = j & 1;
        const uint32_t sb_addr = lane_addr + S2_COL + (2 * x + b) * BN2;     // scores, then probabilities
        if (!mbar_wait(smem_u32(&bars->sd_full[x][b]), (uint32_t)((j >> 1) & 1))) { ok = false; break; }
        tc_fence_after();
        const int key0 = (j0 + j) * BN2;
        const bool need_mask = key0 + BN2 - 1 > ctx + tok0;
        uint32_t v[64];
        tmem_ld64(sb_addr, v);
        tmem_ld_wait();
        float mx = -INFINITY;
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < 64; i += 2) mx = fmaxf(mx, fmaxf(__uint_as_float(v[i]), __uint_as_float(v[i + 1])));
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            if (key0 + i > lim) v[i] = 0xff800000u;      // -inf: its probability is 0
            mx = fmaxf(mx, __uint_as_float(v[i]));
          }
        }
        mx *= sl2;
        const bool grow = mx > m + 8.0f || (m == -INFINITY && mx > -INFINITY);
        float alpha = 1.0f;
        if (grow) {
          alpha = fast_exp2(m - mx);
          m = mx;
        }
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          if (!mbar_wait(smem_u32(&bars->pv_done[x][(j - 1) & 1]), (uint32_t)(((j - 1) >> 1) & 1))) { ok = false; break; }
          tc_fence_after();
          rescale_output(alpha);
          l *= alpha;
        }
        const float m_use = m == -INFINITY ? 0.f : m;
        float sum = 0.f;
        uint32_t w[32];
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(v[i]), sl2, -m_use));
          const float p1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), sl2, -m_use));
          sum += p0;
          sum += p1;
          w[i >> 1] = pack2(p0, p1);
        }
        tmem_st32(sb_addr, w);                           // over the first half of the tile's own scores
        tmem_st_wait();
        l += sum;
        if (key0 + BN2 > kend_all && !zero_stale_values(j, key0)) { ok = false; break; }
        tc_fence_before();
        mbar_arrive(smem_u32(&bars->pd_full[x][b]));
      }
      if (ok && nt > 0) ok = mbar_wait(smem_u32(&bars->pv_done[x][(nt - 1) & 1]), (uint32_t)(((nt - 1) >> 1) & 1));
    } else {
    for (int j = 0; j < nt && ok; ++j) {
      if (!mbar_wait(smem_u32(&bars->s_full[x]), (uint32_t)(j & 1))) { ok = false; break; }
      tc_fence_after();
      const int key0 = (j0 + j) * BN2;
      const bool need_mask = key0 + BN2 - 1 > ctx + tok0;     // some row of the tile does not see the whole tile
      // first pass: the row's maximum (tiles left of the diagonal need no mask)
      float mx = -INFINITY;
      if (!need_mask) {
#pragma unroll
        for (int c = 0; c < BN2; c += 64) {
          uint32_t v[64];
          tmem_ld64(s_addr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 64; i += 2) mx = fmaxf(mx, fmaxf(__uint_as_float(v[i]), __uint_as_float(v[i + 1])));
        }
      } else {
#pragma unroll
        for (int c = 0; c < BN2; c += 64) {
          uint32_t v[64];
          tmem_ld64(s_addr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 64; ++i) mx = fmaxf(mx, key0 + c + i <= lim ? __uint_as_float(v[i]) : -INFINITY);
        }
      }
      mx *= sl2;                                         // scale > 0: the maximum commutes with it
      const bool grow = mx > m + 8.0f || (m == -INFINITY && mx > -INFINITY);
      float alpha = 1.0f;
      if (grow) {
        alpha = fast_exp2(m - mx);                       // 0 while nothing has been summed
        m = mx;
      }
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        if (!mbar_wait(smem_u32(&bars->o_full[x]), (uint32_t)((j - 1) & 1))) { ok = false; break; }
        tc_fence_after();
        rescale_output(alpha);
        l *= alpha;
      }
      const float m_use = m == -INFINITY ? 0.f : m;
      if (!mbar_wait(smem_u32(&bars->p_empty[x]), (uint32_t)((j & 1) ^ 1))) { ok = false; break; }
      // second pass: probabilities to tensor memory, two keys per column: the P V product reads
      // them from there, and shared memory carries K, V and Q only
      float sum = 0.f;
      auto second_pass = [&](auto masked) {
        constexpr bool MASKED = decltype(masked)::value;
#pragma unroll
        for (int c = 0; c < BN2; c += 64) {
          uint32_t v[64];
          tmem_ld64(s_addr + c, v);
          tmem_ld_wait();
          uint32_t w[32];
#pragma unroll
          for (int i = 0; i < 64; i += 2) {
            float sc0 = fmaf(__uint_as_float(v[i]), sl2, -m_use), sc1 = fmaf(__uint_as_float(v[i + 1]), sl2, -m_use);
            if (MASKED && key0 + c + i > lim) sc0 = -INFINITY;
            if (MASKED && key0 + c + i + 1 > lim) sc1 = -INFINITY;
            const float p0 = fast_exp2(sc0), p1 = fast_exp2(sc1);
            sum += p0;
            sum += p1;
            w[i >> 1] = pack2(p0, p1);
          }
          tmem_st32(p_addr + (c >> 1), w);
        }
        tmem_st_wait();
      };
      if (need_mask) second_pass(std::true_type{});
      else second_pass(std::false_type{});
      tc_fence_before();
      mbar_arrive(smem_u32(&bars->s_empty[x]));          // the scores have been read twice: free for tile j + 1
      l += sum;
      if (key0 + BN2 > kend_all && !zero_stale_values(j, key0)) { ok = false; break; }
      tc_fence_before();
      mbar_arrive(smem_u32(&bars->p_full[x]));
    }
    if (ok && nt > 0) ok = mbar_wait(smem_u32(&bars->o_full[x]), (uint32_t)((nt - 1) & 1));
    }
    if (!ok) {
      if (lane == 0) fmx_set_status(status, FMX_WAIT_EXPIRED, 23, blockIdx.x);
    } else if (ksplits > 1) {
      // the partial of this split: outputs at the scale m (log2 domain) with their sum l; no tiles: nothing seen
      if (nt > 0) tc_fence_after();
      const long long slot = ((long long)split * T + (t0 + tok0 + tok)) * nh + head;
      float* po = part_o + slot * HD;
      if (rvalid) {
        part_ml[slot * 2] = nt > 0 ? m : -INFINITY;
        part_ml[slot * 2 + 1] = nt > 0 ? l : 0.f;
      }
      if (nt > 0) {
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          uint32_t v[32];
          tmem_ld32(o_addr + c, v);                      // the whole warp loads; valid rows store
          tmem_ld_wait();
          if (rvalid) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              *reinterpret_cast<uint4*>(po + c + i) = make_uint4(v[i], v[i + 1], v[i + 2], v[i + 3]);
          }
        }
      }
    } else if (nt > 0) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      bf16* op = out + ((long long)(t0 + tok0 + tok) * nh + head) * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        uint32_t v[32];
        tmem_ld32(o_addr + c, v);                        // the whole warp loads; valid rows store
        tmem_ld_wait();
        if (rvalid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack2(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
            w.y = pack2(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
            w.z = pack2(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
            w.w = pack2(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
            *reinterpret_cast<uint4*>(op + c + i) = w;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

// out[t, h, :] = sum over the shares of their outputs, brought to a common scale, over the sum of their sums.  One block
// per token: the shares' scales and sums of all heads go to shared memory first, then every thread walks (head, dim)
// pairs with consecutive threads on consecutive dims.
constexpr int COMBINE_THREADS = 256, COMBINE_MAX_HEADS = 256;
__global__ void __launch_bounds__(COMBINE_THREADS)
attn_prefill_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                            const int* __restrict__ row_start, bf16* out, int rows, int nh, int T, int ksplits) {
  __shared__ float weight[4][COMBINE_MAX_HEADS];         // per share and head: 2^(m - M) / L
  pdl_wait();
  const int t = (int)blockIdx.x + row_start[0];          // tokens of the launch's rows only
  if (t >= row_start[rows]) return;
  for (int h = threadIdx.x; h < nh; h += COMBINE_THREADS) {
    const long long idx = (long long)t * nh + h;
    float m[4], l[4], M = -INFINITY;
#pragma unroll
    for (int sp = 0; sp < 4; ++sp) {
      const bool on = sp < ksplits;
      m[sp] = on ? part_ml[((long long)sp * T * nh + idx) * 2] : -INFINITY;
      l[sp] = on ? part_ml[((long long)sp * T * nh + idx) * 2 + 1] : 0.f;
      M = fmaxf(M, m[sp]);
    }
    const float Mu = M == -INFINITY ? 0.f : M;
    float L = 0.f;
#pragma unroll
    for (int sp = 0; sp < 4; ++sp) L += exp2f(m[sp] - Mu) * l[sp];
    const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
    for (int sp = 0; sp < 4; ++sp) weight[sp][h] = exp2f(m[sp] - Mu) * inv;
  }
  __syncthreads();
  const int per_token = nh * HD;
  for (int e = 4 * threadIdx.x; e < per_token; e += 4 * COMBINE_THREADS) {       // HD is a multiple of 16: four dims of one head
    const int h = e / HD;
    const long long at = (long long)t * per_token + e;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sp = 0; sp < ksplits; ++sp) {
      const float w = weight[sp][h];
      if (w > 0.f) {                                     // a share that saw nothing left its outputs unwritten
        const float4 v = *reinterpret_cast<const float4*>(part_o + (long long)sp * T * per_token + at);
        acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
      }
    }
    uint2 packed;
    packed.x = pack2(acc.x, acc.y);
    packed.y = pack2(acc.z, acc.w);
    *reinterpret_cast<uint2*>(out + at) = packed;
  }
}
}  // namespace two

}  // namespace

// 1 when this head size has the tensor-memory kernel.
FMX_EXPORT int fmx_attn_prefill_tc_available() { return 1; }

// As fmx_attn_prefill, without a window, for up to 16 query heads per kv head and a page size
// that divides 128 and is at least 8.  q rows (tokens) are T; the out-of-range part of the
// last query tile reads as zeros.  variant 1: one query tile per CTA; otherwise two (where the
// page size divides that kernel's key tile: 128 keys at head size 64, 64 at 128).
// How many CTAs share the keys of a pair of query tiles: 1 unless the grid of the two-tile kernel would leave more than
// half of the SMs idle and every share still has 768 keys to walk; 2 or 4.  One 512-token portion at head size 64 / 128,
// microseconds: behind 1,024 keys 28 -> 23 / 35 -> 29, behind 4,096 keys 70 -> 45 / 89 -> 58, behind 16,384 keys
// 240 -> 132 / 305 -> 167; with nothing behind it 14 -> 15 / 16 -> 19, which is why short contexts are left alone.
FMX_EXPORT int fmx_attn_prefill_tc_plan_splits(int rows, int max_q_len, int max_ctx_after, int nh, int nkv, int sms) {
  if (sms <= 0) sms = fmx_num_sms();
  if (rows <= 0 || max_q_len <= 0 || nkv <= 0 || nh % nkv || nh > two::COMBINE_MAX_HEADS) return 1;
  const int tok_per_tile = BM / (nh / nkv);
  const long long pairs = (long long)nkv * rows * ((max_q_len + 2 * tok_per_tile - 1) / (2 * tok_per_tile));
  const int tiles = (max_ctx_after + two::BN2 - 1) / two::BN2;
  int s = (int)(sms / (pairs > 0 ? pairs : 1));
  if (s > 4) s = 4;
  while (s > 1 && tiles / s < 768 / two::BN2) --s;      // a share walks at least 768 keys
  if (s == 3) s = 2;                                  // three shares were slower than two wherever they were timed
  return s < 1 ? 1 : s;
}

// Floats of workspace that `ksplits` shares of the keys need for a step of T tokens (0 for one share).
FMX_EXPORT long long fmx_attn_prefill_tc_scratch_floats(int T, int nh, int ksplits) {
  return ksplits <= 1 ? 0 : (long long)ksplits * T * nh * (HD + 2);
}

// ksplits: 0 or 1: every pair of query tiles walks all of its keys; more: that many CTAs share them (the two-tile kernel
// only), their partials in `scratch` (fmx_attn_prefill_tc_scratch_floats), combined by a second kernel.
FMX_EXPORT int fmx_attn_prefill_tc(const void* q, long long q_stride, int T, const void* kv, const int* block_tables,
                                   int bt_stride, const int* row_start, const int* row_ctx, void* out, int rows,
                                   int max_q_len, int nh, int nkv, int page_size, long long num_pages, float scale,
                                   int variant, int* status, int ksplits, float* scratch, long long scratch_floats,
                                   cudaStream_t stream) {
  if (rows == 0 || max_q_len == 0) return 0;
  if (ksplits < 1) ksplits = 1;
  if (ksplits > 4 || (ksplits > 1 && nh > two::COMBINE_MAX_HEADS))
    return fmx_fail("fmx_attn_prefill_tc: at most 4 shares of the keys and %d heads with them (asked: %d, %d)", two::COMBINE_MAX_HEADS, ksplits, nh);
  if (ksplits > 1 && (scratch == nullptr || scratch_floats < fmx_attn_prefill_tc_scratch_floats(T, nh, ksplits)))
    return fmx_fail("fmx_attn_prefill_tc: %d shares of the keys need %lld floats of workspace, %lld given", ksplits,
                    fmx_attn_prefill_tc_scratch_floats(T, nh, ksplits), scratch_floats);
  if (rows < 0 || nh <= 0 || nkv <= 0 || nh % nkv) return fmx_fail("fmx_attn_prefill_tc: bad sizes rows=%d nh=%d nkv=%d", rows, nh, nkv);
  const int rep = nh / nkv;
  if (rep > 16) return fmx_fail("fmx_attn_prefill_tc: %d query heads per kv head is above 16", rep);
  if (page_size < 8 || BN % page_size) return fmx_fail("fmx_attn_prefill_tc: a page of %d tokens does not tile 128 keys", page_size);
  if (rows > 65535 || nkv > 65535) return fmx_fail("fmx_attn_prefill_tc: too many rows or kv heads for one launch");
  if ((long long)max_q_len * (nh / nkv) > 65535LL * BM)
    return fmx_fail("fmx_attn_prefill_tc: %d query tokens in one row are too many for one launch", max_q_len);
  if (q_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)kv & 15)) return fmx_fail("fmx_attn_prefill_tc: q and the cache must be 16-byte aligned");
  EncodeTiledFn enc = encode_fn();
  if (enc == nullptr) return fmx_fail("fmx_attn_prefill_tc: cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap map_q, map_kv;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)nh, (cuuint64_t)T};
    const cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)q_stride * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)rep, (cuuint32_t)(BM / rep)};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult rc = enc(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fmx_fail("fmx_attn_prefill_tc: encoding the query map failed with code %d", (int)rc);
  }
  const long long kv_rows = num_pages * 2 * nkv * page_size;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)kv_rows};
    const cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult rc = enc(&map_kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(kv), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fmx_fail("fmx_attn_prefill_tc: encoding the cache map failed with code %d", (int)rc);
  }
  if (kv_rows >= 2147483647LL) return fmx_fail("fmx_attn_prefill_tc: the cache has too many rows for a 32-bit coordinate");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return fmx_fail("fmx_attn_prefill_tc: %zu bytes of shared memory refused: %s", SMEM_BYTES, cudaGetErrorString(e));
    configured = true;
  }
  const int tok_per_tile = BM / rep;
  // Two query tiles per CTA share every K/V tile and are the faster kernel when the grid fills the GPU.  At head
  // size 64 a grid of at most half the SMs does better with one tile per CTA and twice the CTAs (one 512-token portion
  // with 32 query heads: 64 CTAs 13.8 us, 128 CTAs 11.7; behind 32,768 keys 476 and 394 us); at head size 128 the
  // two-tile kernel wins even then (587 against 803 us).
  const long long pairs = (long long)nkv * rows * ((max_q_len + 2 * tok_per_tile - 1) / (2 * tok_per_tile));
  if (variant == 0 && HD == 64 && ksplits <= 1 && 2 * pairs <= fmx_num_sms()) variant = 1;      // 0: this choice; 1, 2: the caller's
  if (ksplits > 1 && (variant == 1 || two::BN2 % page_size != 0))
    return fmx_fail("fmx_attn_prefill_tc: only the kernel with two query tiles per CTA shares keys out (page size %d)", page_size);
  if (variant != 1 && two::BN2 % page_size == 0) {      // two query tiles per CTA
    static bool configured2 = false;
    if (!configured2) {
      cudaError_t e2 = cudaFuncSetAttribute(two::attn_prefill_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)two::SMEM2);
      if (e2 != cudaSuccess) return fmx_fail("fmx_attn_prefill_tc: %zu bytes of shared memory refused: %s", two::SMEM2,
                                             cudaGetErrorString(e2));
      configured2 = true;
    }
    const long long z = (long long)((max_q_len + 2 * tok_per_tile - 1) / (2 * tok_per_tile)) * ksplits;
    if (z > 65535) return fmx_fail("fmx_attn_prefill_tc: too many query tiles and shares for one launch");
    dim3 grid2(nkv, rows, (unsigned)z);
    float* part_o = scratch;
    float* part_ml = ksplits > 1 ? scratch + (long long)ksplits * T * nh * HD : nullptr;
    cudaError_t e2 = fmx_launch(two::attn_prefill_tc2_kernel, grid2, dim3(two::THREADS2), two::SMEM2, stream, map_q, map_kv,
                                block_tables, bt_stride, row_start, row_ctx, (bf16*)out, nh, nkv, page_size, num_pages,
                                kv_rows, scale, status, ksplits, part_o, part_ml, T);
    if (e2 != cudaSuccess) return fmx_fail("fmx_attn_prefill_tc: launch failed: %s", cudaGetErrorString(e2));
    if (ksplits > 1) {
      e2 = fmx_launch(two::attn_prefill_combine_kernel, dim3((unsigned)T), dim3(two::COMBINE_THREADS), 0, stream,
                      (const float*)part_o, (const float*)part_ml, row_start, (bf16*)out, rows, nh, T, ksplits);
      if (e2 != cudaSuccess) return fmx_fail("fmx_attn_prefill_tc: launching the combining kernel failed: %s", cudaGetErrorString(e2));
    }
    return 0;
  }
  dim3 grid(nkv, rows, (max_q_len + tok_per_tile - 1) / tok_per_tile);
  cudaError_t e = fmx_launch(attn_prefill_tc_kernel, grid, dim3(THREADS), SMEM_BYTES, stream, map_q, map_kv, block_tables,
                             bt_stride, row_start, row_ctx, (bf16*)out, nh, nkv, page_size, num_pages, kv_rows, scale, status);
  if (e != cudaSuccess) return fmx_fail("fmx_attn_prefill_tc: launch failed: %s", cudaGetErrorString(e));
  return 0;
}
#else
#include "common.cuh"
FMX_EXPORT int fmx_attn_prefill_tc_available() { return 0; }
FMX_EXPORT int fmx_attn_prefill_tc_plan_splits(int, int, int, int, int, int) { return 1; }
FMX_EXPORT long long fmx_attn_prefill_tc_scratch_floats(int, int, int) { return 0; }
FMX_EXPORT int fmx_attn_prefill_tc(const void*, long long, int, const void*, const int*, int, const int*, const int*, void*,
                                   int, int, int, int, int, long long, float, int, int*, int, float*, long long, cudaStream_t) {
  return fmx_fail("fmx_attn_prefill_tc: this head size has no tensor-memory attention kernel");
}
#endif
