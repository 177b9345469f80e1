// Paged grouped-query attention in bfloat16 on the tensor cores, for one head size
// (compile with -DFMX_HD=<head size>, a multiple of 16 up to 256).
//
// Two kernels over the same paged cache [page, 2 (k|v), nkv, page_size, hd]:
//
//  * prefill: a block owns 64 "packed" query rows of one request and one kv head.  Packed
//    row i stands for (token i / rep, query head g*rep + i % rep), rep = nh / nkv, so all
//    rows of a block read the same keys and values; each has its own causal limit.  Keys
//    and values stream through shared memory in tiles of 64 keys (cp.async, three stages);
//    scores, running maximum and sum, and the output accumulator are 32-bit (flash-style
//    online softmax).  It takes any mix of rows: portions of prompts and single tokens.
//
//  * decode: every row brings one token.  A block owns (a split of the keys, a kv head, a row).  The keys are
//    the rows of the MMA and up to 8 query heads its columns (S^T = K Q^T, O^T += V^T P^T), so the few heads of
//    a kv head are not padded to 16 rows.  Each of the four warps streams tiles of its own through its own ring
//    in shared memory (cp.async, no block barrier in the loop); the warps merge at the end.  The splits of a
//    (row, kv head) are either one thread-block cluster, whose first block adds up the partials (maximum, sum,
//    accumulator) through distributed shared memory behind the hardware's cluster barrier, or write their
//    partials to a workspace, where the block that draws the row's last ticket (or a second kernel) combines
//    them.  No block spins on a flag: there is nothing to hang.
//
// Keys out of sight (beyond a row's position, before its window, or in no page) are
// zero-filled in shared memory and masked, never read from the cache.
#include <mutex>
#include <math.h>
#include "common.cuh"

#ifndef FMX_HD
#error "compile with -DFMX_HD=<head size>"
#endif

namespace {
constexpr int HD = FMX_HD;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16, at most 256");
constexpr int KSTEPS = HD / 16;          // k-steps of Q.K^T
constexpr int NT_O = HD / 8;             // 8-wide column tiles of the output
constexpr int BN = 64;                   // keys per tile
constexpr int BM = 64;                   // packed query rows per prefill block
constexpr int ROW = HD + 8;              // padded shared-memory row (elements): conflict-free ldmatrix
constexpr int CHUNKS = HD / 8;           // 16-byte chunks per row
constexpr int TILE = BN * ROW;           // elements of one K (or V) tile
constexpr int THREADS = 128;
constexpr int PREFILL_STAGES = HD <= 128 ? 3 : 2;
constexpr int DECODE_STAGES = HD <= 128 ? 3 : 2;
constexpr int MO_ROW = HD + 4;           // floats in a row of a warp's partial output: heads 2t and 2t + 2 on other banks
// Groups of 16 keys in a warp's decode tile.  Grids of few blocks (batch 1 to 4 with 8 kv heads) are bound by the
// chain of one pass of the loop, not by bandwidth: there a pass takes 32 keys per warp where two blocks of that
// ring still share an SM (head sizes up to 64).  Measured at head size 64, batch 1 over 131,072 keys: 16 keys a
// pass 56.8 us, 32 keys 51.5; batch 8 over 8,192: 28.5 and 28.9.
constexpr int FEW_KG = (2 * 3 * 2 * 4 * 32 * (HD + 8) * 2 <= 226 * 1024) ? 2 : 1;
constexpr float LOG2E = 1.4426950408889634f;
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the special-function unit (about two units in the last place; -inf gives 0).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

struct Cache {
  const bf16* kv;
  const int* bt;          // this row's block table
  int bt_len;
  int nkv, page_size;
  long long num_pages;
  int page_shift;         // log2(page_size) when it is a power of two >= 4, else -1
};

__device__ __forceinline__ int page_shift_of(int page_size) {
  return (page_size >= 4 && (page_size & (page_size - 1)) == 0) ? 31 - __clz(page_size) : -1;
}

// Bring keys [k0, k0 + BN) of kv head g into a shared K tile and a shared V tile; keys
// outside [kbeg, kend) or without a page become zeros.  k0 is a multiple of 4.  When the
// page size is a power of two (>= 4), four consecutive keys share a page: one block-table
// read serves eight 16-byte copies.
__device__ __forceinline__ void load_tiles(bf16* kdst, bf16* vdst, const Cache& c, int g, int k0, int kbeg, int kend,
                                           int* status, int where) {
  const long long plane = (long long)c.nkv * c.page_size * HD;          // k plane -> v plane
  const long long page_stride = 2 * plane;
  const bf16* base = c.kv + (long long)g * c.page_size * HD;
  if (c.page_shift >= 0 && k0 >= kbeg && k0 + BN <= kend) {
    // A tile inside the range (all but the first and last of a block): no key needs a test, and what does not
    // depend on the tile (the thread's chunk, its place in the shared tile) folds into the copies' offsets.
    const unsigned kbase = (unsigned)__cvta_generic_to_shared(kdst), vbase = (unsigned)__cvta_generic_to_shared(vdst);
#pragma unroll
    for (int it = 0; it < ((BN / 4) * CHUNKS + THREADS - 1) / THREADS; ++it) {
      const int item = threadIdx.x + it * THREADS;
      if (((BN / 4) * CHUNKS) % THREADS != 0 && item >= (BN / 4) * CHUNKS) break;
      const int rg = item / CHUNKS, ch = item - rg * CHUNKS;
      const int key0 = k0 + 4 * rg;
      const int blk = key0 >> c.page_shift;
      const int page = blk < c.bt_len ? c.bt[blk] : -1;
      const bool have = page >= 0 && page < c.num_pages;
      if (!have) fmx_set_status(status, FMX_BAD_PAGE, page, where);
      const bf16* src = have ? base + page * page_stride + (long long)(key0 & (c.page_size - 1)) * HD + ch * 8 : c.kv;
      const int n = have ? 16 : 0;                     // 0: zeros, and nothing is read (the offsets stay inside page 0)
      const unsigned off = (unsigned)(((4 * rg) * ROW + ch * 8) * 2);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(kbase + off + i * ROW * 2), "l"(src + i * HD), "r"(n));
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(vbase + off + i * ROW * 2), "l"(src + i * HD + plane), "r"(n));
      }
    }
    return;
  }
  if (c.page_shift >= 0) {
    for (int item = threadIdx.x; item < (BN / 4) * CHUNKS; item += THREADS) {
      const int rg = item / CHUNKS, ch = item - rg * CHUNKS;
      const int key0 = k0 + 4 * rg;
      const bool any = key0 + 3 >= kbeg && key0 < kend;
      const bf16* src = c.kv;
      bool have = false;
      if (any) {
        const int blk = key0 >> c.page_shift;
        const int page = blk < c.bt_len ? c.bt[blk] : -1;
        if (page < 0 || page >= c.num_pages) {
          fmx_set_status(status, FMX_BAD_PAGE, page, where);
        } else {
          have = true;
          src = base + page * page_stride + (long long)(key0 & (c.page_size - 1)) * HD + ch * 8;
        }
      }
      bf16* kd = kdst + (4 * rg) * ROW + ch * 8;
      bf16* vd = vdst + (4 * rg) * ROW + ch * 8;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bool valid = have && key0 + i >= kbeg && key0 + i < kend;
        cp_async16(kd + i * ROW, valid ? src + i * HD : c.kv, valid);
        cp_async16(vd + i * ROW, valid ? src + i * HD + plane : c.kv, valid);
      }
    }
    return;
  }
  for (int idx = threadIdx.x; idx < BN * CHUNKS; idx += THREADS) {
    const int r = idx / CHUNKS, ch = idx - r * CHUNKS;
    const int key = k0 + r;
    bool valid = key >= kbeg && key < kend;
    const bf16* src = c.kv;
    if (valid) {
      const int blk = key / c.page_size;
      const int page = blk < c.bt_len ? c.bt[blk] : -1;
      if (page < 0 || page >= c.num_pages) {
        fmx_set_status(status, FMX_BAD_PAGE, page, where);
        valid = false;
      } else {
        src = base + page * page_stride + (long long)(key - blk * c.page_size) * HD + ch * 8;
      }
    }
    cp_async16(kdst + r * ROW + ch * 8, src, valid);
    cp_async16(vdst + r * ROW + ch * 8, valid ? src + plane : c.kv, valid);
  }
}

// S[16 x 8*NT] += Q[16 x HD] . K^T for the key rows [key_row0, key_row0 + 8*NT) of a shared tile.
template <int NT>
__device__ __forceinline__ void qk_tile(float (&s)[NT][4], const unsigned (&q)[KSTEPS][4], const bf16* ks, int key_row0) {
  const int lane = threadIdx.x & 31;
  const int mi = lane >> 3, ri = lane & 7;
#pragma unroll
  for (int k = 0; k < KSTEPS; ++k) {
#pragma unroll
    for (int jp = 0; jp < NT / 2; ++jp) {
      unsigned b0, b1, b2, b3;
      // matrices: (keys 16jp.., hd 16k), (same keys, hd 16k+8), (keys 16jp+8.., hd 16k), (.., hd 16k+8)
      const bf16* p = ks + (key_row0 + 16 * jp + (mi >> 1) * 8 + ri) * ROW + 16 * k + (mi & 1) * 8;
      ldmatrix_x4(b0, b1, b2, b3, p);
      mma_bf16(s[2 * jp], q[k], b0, b1);
      mma_bf16(s[2 * jp + 1], q[k], b2, b3);
    }
  }
}

// O[16 x HD] += P[16 x 16*KT] . V for the key rows [key_row0, ...) of a shared tile; P comes
// as the score fragments of 2*KT column tiles.
template <int KT>
__device__ __forceinline__ void pv_tile(float (&o)[NT_O][4], const float (&p)[2 * KT][4], const bf16* vs, int key_row0) {
  const int lane = threadIdx.x & 31;
  const int mi = lane >> 3, ri = lane & 7;
#pragma unroll
  for (int kk = 0; kk < KT; ++kk) {
    unsigned a[4];
    a[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
    a[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
    a[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
    a[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
    for (int np = 0; np < NT_O / 2; ++np) {
      unsigned b0, b1, b2, b3;
      // matrices: (keys 16kk.., hd 16np), (keys 16kk+8.., hd 16np), (keys 16kk.., hd 16np+8), (keys 16kk+8.., hd 16np+8)
      const bf16* ptr = vs + (key_row0 + 16 * kk + (mi & 1) * 8 + ri) * ROW + 16 * np + (mi >> 1) * 8;
      ldmatrix_x4_trans(b0, b1, b2, b3, ptr);
      mma_bf16(o[2 * np], a, b0, b1);
      mma_bf16(o[2 * np + 1], a, b2, b3);
    }
  }
}

// Mask, then one step of the online softmax over NT column tiles for the two rows (g, g+8)
// a thread holds.  Scores arrive raw; sl2 = scale * log2(e).  m is kept in the scaled
// log2 domain.  `lim[x]`, `lo[x]`: last and first visible key of row x.
template <int NT, bool MASK>
__device__ __forceinline__ void softmax_step(float (&s)[NT][4], float (&m)[2], float (&l)[2], float (&alpha)[2], float sl2,
                                             int key0, const int (&lim)[2], const int (&lo)[2]) {
  const int t = threadIdx.x & 3;
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int x = e >> 1;
      const int key = key0 + 8 * j + 2 * t + (e & 1);
      const float v = (!MASK || (key <= lim[x] && key >= lo[x])) ? s[j][e] * sl2 : -INFINITY;
      s[j][e] = v;
      mx[x] = fmaxf(mx[x], v);
    }
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    mx[x] = fmaxf(mx[x], __shfl_xor_sync(0xffffffffu, mx[x], 1));
    mx[x] = fmaxf(mx[x], __shfl_xor_sync(0xffffffffu, mx[x], 2));
    const float m_new = fmaxf(m[x], mx[x]);
    const float m_use = m_new == -INFINITY ? 0.f : m_new;
    alpha[x] = fast_exp2(m[x] - m_use);
    m[x] = m_new;
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const float p0 = fast_exp2(s[j][2 * x] - m_use), p1 = fast_exp2(s[j][2 * x + 1] - m_use);
      s[j][2 * x] = p0;
      s[j][2 * x + 1] = p1;
      sum += p0 + p1;
    }
    l[x] = l[x] * alpha[x] + sum;          // this thread's share; the quad is summed at the end
  }
}

// ---- decode: keys on the rows ----
// A decode row brings the few query heads of one kv head (4 with Llama's grouping).  With the heads on the 16 rows
// of the MMA three quarters of every product were padding; here the keys are the rows and up to 8 heads the
// columns: S^T = K . Q^T, O^T += V^T . P^T.  Per 16 keys that is HD/16 products for the scores and HD/16 for the
// output (half of what the other orientation took), four scores per thread instead of eight, and an accumulator of
// half the size.  The probabilities leave the score product as its C fragment (keys g, g+8; heads 2t, 2t+1) and
// enter the output product as a B fragment (keys 2t, 2t+1, 2t+8, 2t+9; head g): one movmatrix each way.
__device__ __forceinline__ unsigned movmatrix_trans(unsigned a) {
  unsigned d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}

// s[nh] (16 keys x 8 heads) = K rows [key_row0, +16) of a shared tile . Q^T; q[nh][k]: the B fragments of head
// group nh at k-step k.  Two accumulators take alternate k-steps so that the products do not form one chain.
template <int NH>
__device__ __forceinline__ void qk_keys(float (&s)[NH][4], const unsigned (&q)[NH][KSTEPS][2], const bf16* ks, int key_row0) {
  const int lane = threadIdx.x & 31, mi = lane >> 3, ri = lane & 7;
  // matrices: (keys 0-7, hd 16k), (keys 8-15, hd 16k), (keys 0-7, hd 16k+8), (keys 8-15, hd 16k+8)
  const bf16* p = ks + (key_row0 + (mi & 1) * 8 + ri) * ROW + (mi >> 1) * 8;
  float s2[NH][4];
#pragma unroll
  for (int h = 0; h < NH; ++h)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[h][e] = s2[h][e] = 0.f;
#pragma unroll
  for (int k = 0; k < KSTEPS; ++k) {
    unsigned a[4];
    ldmatrix_x4(a[0], a[1], a[2], a[3], p + 16 * k);
#pragma unroll
    for (int h = 0; h < NH; ++h) {
      if (k & 1) mma_bf16(s2[h], a, q[h][k][0], q[h][k][1]);
      else mma_bf16(s[h], a, q[h][k][0], q[h][k][1]);
    }
  }
#pragma unroll
  for (int h = 0; h < NH; ++h)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[h][e] += s2[h][e];
}

// One step of the online softmax for the heads (2t, 2t+1) of each head group that a thread holds, over the 16 KG keys
// key0 + 16 kg + {g, g+8}; keys outside [kfirst, klast] are masked when MASK.  m, l, alpha are per head and the same
// in the eight lanes that share t (l is each lane's share until the end).  Leaves the probabilities as B fragments.
template <int NH, int KG, bool MASK>
__device__ __forceinline__ void softmax_keys(float (&s)[KG][NH][4], float (&m)[NH][2], float (&l)[NH][2], float (&alpha)[NH][2],
                                             unsigned (&pb)[KG][NH][2], float sl2, int key0, int kfirst, int klast) {
  const int g = (threadIdx.x & 31) >> 2;
  bool ok[KG][2];
#pragma unroll
  for (int kg = 0; kg < KG; ++kg)
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      const int key = key0 + 16 * kg + g + 8 * x;
      ok[kg][x] = !MASK || (key >= kfirst && key <= klast);
    }
#pragma unroll
  for (int h = 0; h < NH; ++h) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float mx = -INFINITY;
#pragma unroll
      for (int kg = 0; kg < KG; ++kg)
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const float v = ok[kg][x] ? s[kg][h][2 * x + j] * sl2 : -INFINITY;
          s[kg][h][2 * x + j] = v;
          mx = fmaxf(mx, v);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float m_new = fmaxf(m[h][j], mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      alpha[h][j] = fast_exp2(m[h][j] - m_use);
      m[h][j] = m_new;
      float sum = 0.f;
#pragma unroll
      for (int kg = 0; kg < KG; ++kg)
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const float pr = fast_exp2(s[kg][h][2 * x + j] - m_use);
          s[kg][h][2 * x + j] = pr;
          sum += pr;
        }
      l[h][j] = l[h][j] * alpha[h][j] + sum;
    }
#pragma unroll
    for (int kg = 0; kg < KG; ++kg) {
      pb[kg][h][0] = movmatrix_trans(pack_bf16(s[kg][h][0], s[kg][h][1]));
      pb[kg][h][1] = movmatrix_trans(pack_bf16(s[kg][h][2], s[kg][h][3]));
    }
  }
}

// o[nh][n] (hd 16n + {g, g+8} x heads 2t, 2t+1) += V^T of the key rows [key_row0, +16) . P^T
template <int NH>
__device__ __forceinline__ void pv_keys(float (&o)[NH][HD / 16][4], const unsigned (&pb)[NH][2], const bf16* vs, int key_row0) {
  const int lane = threadIdx.x & 31, mi = lane >> 3, ri = lane & 7;
  // matrices (transposed on the way): (keys 0-7, hd 16n), (keys 0-7, hd 16n+8), (keys 8-15, hd 16n), (keys 8-15, hd 16n+8)
  const bf16* p = vs + (key_row0 + (mi >> 1) * 8 + ri) * ROW + (mi & 1) * 8;
#pragma unroll
  for (int n = 0; n < HD / 16; ++n) {
    unsigned a[4];
    ldmatrix_x4_trans(a[0], a[1], a[2], a[3], p + 16 * n);
#pragma unroll
    for (int h = 0; h < NH; ++h) mma_bf16(o[h][n], a, pb[h][0], pb[h][1]);
  }
}

// ---- decode: a stream of tiles per warp ----
// Each warp of a decode block walks a quarter of the block's keys by itself: its own ring of tiles of 16 KG keys in
// shared memory, filled by its own lanes' copies and waited for with cp.async.wait_group and a warp barrier.  No
// block barrier stands in the loop, so a warp never waits for a slower one, and the block-table entries of the next
// tile can be read a pass ahead into registers (a block barrier would have made the warp wait for them at once).
template <int KG> struct WarpTile {
  static constexpr int TK = 16 * KG;                        // keys per tile
  static constexpr int ELEMS = TK * ROW;                    // elements of a K (or V) tile
  static constexpr int ITEMS = (TK / 4) * CHUNKS;           // (four keys, one 16-byte chunk)
  static constexpr int PER_LANE = (ITEMS + 31) / 32;
};

template <int KG>
__device__ __forceinline__ void warp_fetch_pages(int (&pg)[WarpTile<KG>::PER_LANE], const Cache& c, int k0) {
  using W = WarpTile<KG>;
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i < W::PER_LANE; ++i) {
    const int item = lane + 32 * i;
    const int blk = (k0 + 4 * (item / CHUNKS)) >> c.page_shift;
    pg[i] = (item < W::ITEMS && blk < c.bt_len) ? c.bt[blk] : -1;
  }
}

// A tile that lies inside the warp's range, pages of a power of two: the entries come in registers.
template <int KG>
__device__ __forceinline__ void warp_tile_inside(bf16* kdst, bf16* vdst, const Cache& c, int g, int k0,
                                                 const int (&pg)[WarpTile<KG>::PER_LANE], int* status, int where) {
  using W = WarpTile<KG>;
  const int lane = threadIdx.x & 31;
  const long long plane = (long long)c.nkv * c.page_size * HD;
  const bf16* base = c.kv + (long long)g * c.page_size * HD;
  const unsigned kbase = (unsigned)__cvta_generic_to_shared(kdst), vbase = (unsigned)__cvta_generic_to_shared(vdst);
#pragma unroll
  for (int i = 0; i < W::PER_LANE; ++i) {
    const int item = lane + 32 * i;
    if (W::ITEMS % 32 != 0 && item >= W::ITEMS) break;
    const int rg = item / CHUNKS, ch = item - rg * CHUNKS;
    const int key0 = k0 + 4 * rg;
    const int page = pg[i];
    const bool have = page >= 0 && page < c.num_pages;
    if (!have) fmx_set_status(status, FMX_BAD_PAGE, page, where);
    const bf16* src = have ? base + page * 2 * plane + (long long)(key0 & (c.page_size - 1)) * HD + ch * 8 : c.kv;
    const int n = have ? 16 : 0;                       // 0: zeros, and nothing is read (the offsets stay inside page 0)
    const unsigned off = (unsigned)(((4 * rg) * ROW + ch * 8) * 2);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(kbase + off + j * ROW * 2), "l"(src + j * HD), "r"(n));
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(vbase + off + j * ROW * 2), "l"(src + j * HD + plane), "r"(n));
    }
  }
}

// Any tile, any page size: keys outside [kbeg, kend) or without a page become zeros.
template <int KG>
__device__ __forceinline__ void warp_tile_any(bf16* kdst, bf16* vdst, const Cache& c, int g, int k0, int kbeg, int kend,
                                              int* status, int where) {
  using W = WarpTile<KG>;
  const int lane = threadIdx.x & 31;
  const long long plane = (long long)c.nkv * c.page_size * HD;
  const bf16* base = c.kv + (long long)g * c.page_size * HD;
  for (int idx = lane; idx < W::TK * CHUNKS; idx += 32) {
    const int rr = idx / CHUNKS, ch = idx - rr * CHUNKS;
    const int key = k0 + rr;
    bool valid = key >= kbeg && key < kend;
    const bf16* src = c.kv;
    if (valid) {
      const int blk = c.page_shift >= 0 ? key >> c.page_shift : key / c.page_size;
      const int page = blk < c.bt_len ? c.bt[blk] : -1;
      if (page < 0 || page >= c.num_pages) {
        fmx_set_status(status, FMX_BAD_PAGE, page, where);
        valid = false;
      } else {
        src = base + page * 2 * plane + (long long)(key - blk * c.page_size) * HD + ch * 8;
      }
    }
    cp_async16(kdst + rr * ROW + ch * 8, src, valid);
    cp_async16(vdst + rr * ROW + ch * 8, valid ? src + plane : c.kv, valid);
  }
}

// ------------------------------------------------------------------------------------ prefill
__global__ void __launch_bounds__(THREADS)
attn_prefill_kernel(const bf16* __restrict__ q, long long q_stride, const bf16* __restrict__ kv,
                    const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ row_start,
                    const int* __restrict__ row_ctx, bf16* __restrict__ out, int nh, int nkv, int page_size,
                    long long num_pages, float scale, int window, int* status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* smem = reinterpret_cast<bf16*>(smem_raw);
  // The last query tiles of a row see the most keys.  Blocks start in the order x, y, z: with the
  // tile index in z the longest blocks of every head and row start first.
  const int r = blockIdx.y, g = blockIdx.x, tile = gridDim.z - 1 - blockIdx.z;
  const int rep = nh / nkv;
  const int t0 = row_start[r], q_len = row_start[r + 1] - t0, ctx = row_ctx[r];
  const int n_packed = q_len * rep;
  const int prow0 = tile * BM;
  if (prow0 >= n_packed || ctx < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  const Cache c{kv, block_tables + (long long)r * bt_stride, bt_stride, nkv, page_size, num_pages,
                page_shift_of(page_size)};

  // the two packed rows of this thread
  int prow[2], tok[2], head[2], lim[2], lo[2];
  bool rvalid[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    prow[x] = prow0 + warp * 16 + gq + 8 * x;
    rvalid[x] = prow[x] < n_packed;
    const int pr = rvalid[x] ? prow[x] : n_packed - 1;
    tok[x] = pr / rep;
    head[x] = g * rep + pr - tok[x] * rep;
    lim[x] = rvalid[x] ? ctx + tok[x] : -1;
    lo[x] = window > 0 ? max(0, ctx + tok[x] - window + 1) : 0;
  }
  // query fragments, straight from global memory
  unsigned qf[KSTEPS][4];
#pragma unroll
  for (int k = 0; k < KSTEPS; ++k)
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      const bf16* qp = q + (long long)(t0 + tok[x]) * q_stride + (long long)head[x] * HD + 16 * k + 2 * tq;
      qf[k][x] = rvalid[x] ? *reinterpret_cast<const unsigned*>(qp) : 0u;
      qf[k][x + 2] = rvalid[x] ? *reinterpret_cast<const unsigned*>(qp + 8) : 0u;
    }

  // keys this block needs: from the first row's window start to the last row's position
  const int first_tok = prow0 / rep;
  const int last_tok = (min(prow0 + BM, n_packed) - 1) / rep;
  const int kbeg = window > 0 ? max(0, ctx + first_tok - window + 1) : 0;
  const int kend = ctx + last_tok + 1;
  const int kstart = kbeg & ~3;                       // tiles start on a multiple of 4 keys
  const int n_tiles = (kend - kstart + BN - 1) / BN;
  const float sl2 = scale * LOG2E;
  // what every row of this warp sees for sure: keys from the last row's window start up to
  // the first row's position; tiles inside that span need no mask
  const int wfirst = min(prow0 + warp * 16, n_packed - 1) / rep, wlast = min(prow0 + warp * 16 + 15, n_packed - 1) / rep;
  const bool warp_full = prow0 + warp * 16 + 15 < n_packed;
  const int sure_lo = window > 0 ? max(0, ctx + wlast - window + 1) : 0;
  const int sure_hi = ctx + wfirst;

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[NT_O][4];
#pragma unroll
  for (int n = 0; n < NT_O; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[n][e] = 0.f;

  auto stage_k = [&](int s) { return smem + (size_t)s * 2 * TILE; };
  auto stage_v = [&](int s) { return smem + (size_t)s * 2 * TILE + TILE; };
#pragma unroll
  for (int s = 0; s < PREFILL_STAGES - 1; ++s) {
    if (s < n_tiles) load_tiles(stage_k(s), stage_v(s), c, g, kstart + s * BN, kbeg, kend, status, r);
    cp_async_commit();
  }
  for (int it = 0; it < n_tiles; ++it) {
    cp_async_wait<PREFILL_STAGES - 2>();
    __syncthreads();
    const int nx = it + PREFILL_STAGES - 1;
    if (nx < n_tiles)
      load_tiles(stage_k(nx % PREFILL_STAGES), stage_v(nx % PREFILL_STAGES), c, g, kstart + nx * BN, kbeg, kend, status, r);
    cp_async_commit();
    const bf16* ks = stage_k(it % PREFILL_STAGES);
    const bf16* vs = stage_v(it % PREFILL_STAGES);
    float s[BN / 8][4];
#pragma unroll
    for (int j = 0; j < BN / 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
    qk_tile<BN / 8>(s, qf, ks, 0);
    float alpha[2];
    const int tk0 = kstart + it * BN;
    if (warp_full && tk0 >= sure_lo && tk0 + BN - 1 <= sure_hi)
      softmax_step<BN / 8, false>(s, m, l, alpha, sl2, tk0, lim, lo);
    else
      softmax_step<BN / 8, true>(s, m, l, alpha, sl2, tk0, lim, lo);
#pragma unroll
    for (int n = 0; n < NT_O; ++n) {
      o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
      o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
    }
    pv_tile<BN / 16>(o, s, vs, 0);
  }
  cp_async_wait<0>();
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    l[x] += __shfl_xor_sync(0xffffffffu, l[x], 1);
    l[x] += __shfl_xor_sync(0xffffffffu, l[x], 2);
    if (!rvalid[x]) continue;
    const float inv = l[x] > 0.f ? 1.0f / l[x] : 0.f;
    bf16* op = out + ((long long)(t0 + tok[x]) * nh + head[x]) * HD + 2 * tq;
#pragma unroll
    for (int n = 0; n < NT_O; ++n)
      *reinterpret_cast<unsigned*>(op + 8 * n) = pack_bf16(o[n][2 * x] * inv, o[n][2 * x + 1] * inv);
  }
}

// ---- the splits of a row as one thread-block cluster ----
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A float of block `rank` of this cluster, at the place where this block has `local`.
__device__ __forceinline__ float ld_cluster(const float* local, unsigned rank) {
  unsigned remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((unsigned)__cvta_generic_to_shared(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}
constexpr int MAX_CLUSTER = 8;           // splits that can be one cluster (the portable size; clusters of 9 placed badly:
                                         // batch 8 over 8,192 keys at head size 64 38.6 us against 27.8 through tickets)

// ------------------------------------------------------------------------------------ decode
// part_o: [R, nkv, splits, 16, HD] float; part_ml: [R, nkv, splits, 16, 2] float (max in the
// scaled log2 domain, sum).  With one split the output is written directly.
template <int STAGES, int NH, int KG>
__global__ void __launch_bounds__(THREADS)
attn_decode_kernel(const bf16* q, long long q_stride, const bf16* kv, const int* block_tables, int bt_stride,
                   const int* row_start, const int* positions, bf16* out, float* part_o, float* part_ml, int nh, int nkv,
                   int page_size, long long num_pages, float scale, int window, int* status, int* tickets,
                   const float* __restrict__ inv_freq, int rot, int interleaved, int rope_mode, int clustered) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* smem = reinterpret_cast<bf16*>(smem_raw);
  const int split = blockIdx.x, splits = gridDim.x, g = blockIdx.y, r = blockIdx.z;
  const int rep = nh / nkv;
  // Row starts, positions and block tables are in place before the step's first kernel runs.
  const int t = row_start[r];
  const int pos = positions[t];                      // -1 for a padding row: no keys at all
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  Cache c{kv, block_tables + (long long)r * bt_stride, bt_stride, nkv, page_size, num_pages,
          page_shift_of(page_size)};

  const int lo_key = window > 0 ? max(0, pos - window + 1) : 0;
  const int n_keys = max(0, pos + 1 - lo_key);
  using W = WarpTile<KG>;
  int per = (n_keys + splits - 1) / splits;
  per = (per + 4 * W::TK - 1) / (4 * W::TK) * (4 * W::TK);
  const int kbeg = lo_key + split * per;
  const int kend = min(pos + 1, kbeg + per);
  // This warp's keys [rbeg, rend) and its tiles of 16 KG keys, which start on a multiple of four keys.  With the
  // small tile the block's tiles go round the warps, which then walk through the same pages side by side (batch 8
  // over 8,192 keys at head size 64: 27.8 us against 28.8); with the large tile of the grids of few blocks each warp
  // has a quarter of the keys to itself (batch 1 over 131,072 keys: 51.2 us against 58.2).
  constexpr bool QUARTERS = KG > 1;
  const int rbeg = QUARTERS ? kbeg + warp * (per / 4) : kbeg;
  const int rend = QUARTERS ? min(kend, rbeg + per / 4) : kend;
  const int rstart = rbeg & ~3;
  const int r_tiles = rend > rbeg ? (rend - rstart + W::TK - 1) / W::TK : 0;
  const int n_tiles = QUARTERS ? r_tiles : (r_tiles > warp ? (r_tiles - warp + 3) / 4 : 0);
  auto tile_key = [&](int tile) { return rstart + (QUARTERS ? tile : 4 * tile + warp) * W::TK; };
  const bool pow2 = c.page_shift >= 0;

  bf16* ring = smem + (size_t)warp * STAGES * 2 * W::ELEMS;
  auto stage_k = [&](int s) { return ring + (size_t)s * 2 * W::ELEMS; };
  auto stage_v = [&](int s) { return ring + (size_t)s * 2 * W::ELEMS + W::ELEMS; };
  int pg[W::PER_LANE];
  // Tile `tile` into its stage; pages of a power of two and a tile inside the range take the short path, with the
  // table entries that `pg` holds when the caller read them ahead.
  auto issue = [&](int tile, bool have_pg) {
    const int k0 = tile_key(tile);
    bf16* kd = stage_k(tile % STAGES);
    bf16* vd = stage_v(tile % STAGES);
    if (pow2 && k0 >= rbeg && k0 + W::TK <= rend) {
      if (!have_pg) warp_fetch_pages<KG>(pg, c, k0);
      warp_tile_inside<KG>(kd, vd, c, g, k0, pg, status, r);
    } else {
      warp_tile_any<KG>(kd, vd, c, g, k0, rbeg, rend, status, r);
    }
  };
  // Keys before this row's new one were written by earlier steps: tiles that end before it are
  // fetched while the kernel ahead (which writes the new key and the queries) is still running.
  int fetched = 0;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (fetched == s && s < n_tiles && min(rend, tile_key(s) + W::TK) <= pos) {
      issue(s, false);
      fetched = s + 1;
    }
  }
  // The last stage of a ring is free until the first pass of the loop below: with rotation in
  // this kernel the first warp's holds the rotated queries and the row's sines and cosines meanwhile.
  // Those depend on the position alone, so they too are ready before the kernel ahead has finished.
  bf16* q_rot = smem + (size_t)(STAGES - 1) * 2 * W::ELEMS;        // [16][HD]
  float* rope_sin = reinterpret_cast<float*>(q_rot + 16 * HD);
  float* rope_cos = rope_sin + HD / 2;
  static_assert(16 * HD * 2 + HD * 4 <= 2 * W::ELEMS * 2, "the rotated queries must fit one stage of a warp");
  const int half = rot / 2;
  if (rope_mode > 0) {
    const float fpos = (float)pos;
    for (int j = threadIdx.x; j < half; j += THREADS) sincosf(fpos * inv_freq[j], &rope_sin[j], &rope_cos[j]);
    __syncthreads();
  }
  pdl_wait();

  const bf16* qbase = q + (long long)t * q_stride + (long long)g * rep * HD;
  long long qhead_stride = HD;
  if (rope_mode > 0) {
    // q, k and v arrive as the projection left them: rotate the queries into shared memory, and
    // let the block whose keys include the row's new one rotate that key and store it and
    // its value in the cache, as the separate kernel would have.
    const bf16* row = q + (long long)t * q_stride;
    for (int it = threadIdx.x; it < rep * (HD / 2); it += THREADS) {
      const int h = it / (HD / 2), j = it - h * (HD / 2);
      const bf16* src = qbase + (long long)h * HD;
      bf16* dst = q_rot + h * HD;
      if (j < half) {
        const int i0 = interleaved ? 2 * j : j, i1 = interleaved ? 2 * j + 1 : j + half;
        float x, y;
        rope_pair(__bfloat162float(src[i0]), __bfloat162float(src[i1]), rope_sin[j], rope_cos[j], x, y);
        dst[i0] = __float2bfloat16_rn(x);
        dst[i1] = __float2bfloat16_rn(y);
      } else {                                       // beyond the rotated part: two elements per item
        const int e = rot + 2 * (j - half);
        dst[e] = src[e];
        dst[e + 1] = src[e + 1];
      }
    }
    if (rope_mode == 1 && pos >= 0 && kbeg <= pos && pos < kend) {
      const int blk = c.page_shift >= 0 ? pos >> c.page_shift : pos / page_size;
      const int page = blk < bt_stride ? c.bt[blk] : -1;
      if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) fmx_set_status(status, FMX_BAD_PAGE, page, r);
      } else {
        const int off = pos - blk * page_size;
        const bf16* ksrc = row + (long long)(nh + g) * HD;
        const bf16* vsrc = row + (long long)(nh + nkv + g) * HD;
        bf16* kdst = const_cast<bf16*>(kv) + ((((long long)page * 2 + 0) * nkv + g) * page_size + off) * HD;
        bf16* vdst = const_cast<bf16*>(kv) + ((((long long)page * 2 + 1) * nkv + g) * page_size + off) * HD;
        for (int j = threadIdx.x; j < HD / 2; j += THREADS) {
          if (j < half) {
            const int i0 = interleaved ? 2 * j : j, i1 = interleaved ? 2 * j + 1 : j + half;
            float x, y;
            rope_pair(__bfloat162float(ksrc[i0]), __bfloat162float(ksrc[i1]), rope_sin[j], rope_cos[j], x, y);
            kdst[i0] = __float2bfloat16_rn(x);
            kdst[i1] = __float2bfloat16_rn(y);
          } else {
            const int e = rot + 2 * (j - half);
            kdst[e] = ksrc[e];
            kdst[e + 1] = ksrc[e + 1];
          }
          vdst[2 * j] = vsrc[2 * j];
          vdst[2 * j + 1] = vsrc[2 * j + 1];
        }
        __threadfence();                             // the tile loads below read the new key through L2
      }
    }
    __syncthreads();
    qbase = q_rot;
  }

  // the queries as B fragments: head 8 h + gq, k = 16 k + 2 tq (+8)
  unsigned qf[NH][KSTEPS][2];
#pragma unroll
  for (int h = 0; h < NH; ++h) {
    const int head = 8 * h + gq;
    const bool ok = head < rep;
    const bf16* qp = qbase + (long long)(ok ? head : 0) * qhead_stride + 2 * tq;
#pragma unroll
    for (int k = 0; k < KSTEPS; ++k) {
      qf[h][k][0] = ok ? *reinterpret_cast<const unsigned*>(qp + 16 * k) : 0u;
      qf[h][k][1] = ok ? *reinterpret_cast<const unsigned*>(qp + 16 * k + 8) : 0u;
    }
  }
  const float sl2 = scale * LOG2E;
  float m[NH][2], l[NH][2];
  float o[NH][HD / 16][4];
#pragma unroll
  for (int h = 0; h < NH; ++h) {
    m[h][0] = m[h][1] = -INFINITY;
    l[h][0] = l[h][1] = 0.f;
#pragma unroll
    for (int n = 0; n < HD / 16; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[h][n][e] = 0.f;
  }

  if (rope_mode > 0) __syncthreads();                // every warp has its queries before the first warp's ring fills up
  // the groups of the pipeline: tile s is in group s, whether it went out before the wait or not
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s >= fetched && s < n_tiles) issue(s, false);
    cp_async_commit();
  }
  int pg_tile = -1;                                  // the tile whose table entries pg holds
  if (pow2 && STAGES - 1 < n_tiles) {
    warp_fetch_pages<KG>(pg, c, tile_key(STAGES - 1));
    pg_tile = STAGES - 1;
  }
  for (int it = 0; it < n_tiles; ++it) {
    cp_async_wait<STAGES - 2>();
    __syncwarp();                                    // every lane's copies of tile `it` have landed; tile it - 1 is read
    const int nx = it + STAGES - 1;
    if (nx < n_tiles) {
      issue(nx, pg_tile == nx);
      if (pow2 && nx + 1 < n_tiles) {
        warp_fetch_pages<KG>(pg, c, tile_key(nx + 1));
        pg_tile = nx + 1;
      }
    }
    cp_async_commit();
    const bf16* ks = stage_k(it % STAGES);
    const bf16* vs = stage_v(it % STAGES);
    float s[KG][NH][4], alpha[NH][2];
    unsigned pb[KG][NH][2];
#pragma unroll
    for (int kg = 0; kg < KG; ++kg) qk_keys<NH>(s[kg], qf, ks, 16 * kg);
    const int wk0 = tile_key(it);
    if (wk0 >= rbeg && wk0 + W::TK <= rend)
      softmax_keys<NH, KG, false>(s, m, l, alpha, pb, sl2, wk0, rbeg, rend - 1);
    else
      softmax_keys<NH, KG, true>(s, m, l, alpha, pb, sl2, wk0, rbeg, rend - 1);
#pragma unroll
    for (int h = 0; h < NH; ++h)
#pragma unroll
      for (int n = 0; n < HD / 16; ++n) {
        o[h][n][0] *= alpha[h][0]; o[h][n][1] *= alpha[h][1];
        o[h][n][2] *= alpha[h][0]; o[h][n][3] *= alpha[h][1];
      }
#pragma unroll
    for (int kg = 0; kg < KG; ++kg) pv_keys<NH>(o, pb[kg], vs, 16 * kg);
  }
  cp_async_wait<0>();
  __syncthreads();                                   // the tiles are done with; reuse the memory
  pdl_trigger();                                     // the block's loads are done: room for the next kernel's

  // merge the four warps: each leaves (m, l, o) of its up to 16 heads
  float* mo = reinterpret_cast<float*>(smem_raw);    // [4][16][MO_ROW]
  float* mml = mo + 4 * 16 * MO_ROW;                 // [4][16][2]
  float* fin_o = mml + 4 * 16 * 2;                   // [16][HD]: the block's partial, where its cluster reads it
  float* fin_ml = fin_o + 16 * HD;                   // [16][2]
#pragma unroll
  for (int h = 0; h < NH; ++h)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float lj = l[h][j];                            // the lanes that share tq hold the shares of this head's sum
      lj += __shfl_xor_sync(0xffffffffu, lj, 4);
      lj += __shfl_xor_sync(0xffffffffu, lj, 8);
      lj += __shfl_xor_sync(0xffffffffu, lj, 16);
      const int row = 8 * h + 2 * tq + j;
      float* dst = mo + ((size_t)warp * 16 + row) * MO_ROW + gq;
#pragma unroll
      for (int n = 0; n < HD / 16; ++n) {
        dst[16 * n] = o[h][n][j];
        dst[16 * n + 8] = o[h][n][2 + j];
      }
      if (gq == 0) {
        mml[(warp * 16 + row) * 2] = m[h][j];
        mml[(warp * 16 + row) * 2 + 1] = lj;
      }
    }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rep * HD; idx += THREADS) {
    const int row = idx / HD, d = idx - row * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, mml[(w * 16 + row) * 2]);
    const float Mu = M == -INFINITY ? 0.f : M;
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(mml[(w * 16 + row) * 2] - Mu);
      L += f * mml[(w * 16 + row) * 2 + 1];
      acc += f * mo[((size_t)w * 16 + row) * MO_ROW + d];
    }
    if (splits == 1) {
      out[((long long)t * nh + g * rep + row) * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    } else if (clustered) {
      fin_o[row * HD + d] = acc;
      if (d == 0) {
        fin_ml[row * 2] = M;
        fin_ml[row * 2 + 1] = L;
      }
    } else {
      const long long pi = (((long long)r * nkv + g) * splits + split) * 16 + row;
      __stcg(&part_o[pi * HD + d], acc);
      if (d == 0) {
        __stcg(&part_ml[pi * 2], M);
        __stcg(&part_ml[pi * 2 + 1], L);
      }
    }
  }
  if (splits == 1) return;
  if (clustered) {
    // The splits of this (row, kv head) are the blocks of one cluster (the split is the rank): their partials stay
    // in shared memory, the cluster's barrier stands where the others write to L2, fence and draw a ticket, and the
    // first block reads them through distributed shared memory, in split order.  Nobody leaves before it has.
    cluster_sync_all();
    if (split == 0) {
      for (int idx = threadIdx.x; idx < rep * HD; idx += THREADS) {
        const int row = idx / HD, d = idx - row * HD;
        float ms[MAX_CLUSTER], ls[MAX_CLUSTER], os[MAX_CLUSTER];
#pragma unroll
        for (int sp = 0; sp < MAX_CLUSTER; ++sp) {
          const bool on = sp < splits;
          ms[sp] = on ? ld_cluster(fin_ml + row * 2, sp) : -INFINITY;
          ls[sp] = on ? ld_cluster(fin_ml + row * 2 + 1, sp) : 0.f;
          os[sp] = on ? ld_cluster(fin_o + row * HD + d, sp) : 0.f;
        }
        float M = -INFINITY;
#pragma unroll
        for (int sp = 0; sp < MAX_CLUSTER; ++sp) M = fmaxf(M, ms[sp]);
        const float Mu = M == -INFINITY ? 0.f : M;
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int sp = 0; sp < MAX_CLUSTER; ++sp) {
          const float f = exp2f(ms[sp] - Mu);        // 0 for the splits that are not there
          L += f * ls[sp];
          acc += f * os[sp];
        }
        out[((long long)t * nh + g * rep + row) * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
      }
    }
    cluster_sync_all();
    return;
  }
  if (tickets == nullptr) return;
  // The block that draws the last ticket of this (row, kv head) combines the splits, in split
  // order.  Nobody waits: the others are done once their partial is written.
  __shared__ int drew_last;
  __syncthreads();                                   // the block's partial is written ...
  if (threadIdx.x == 0) {
    __threadfence();                                 // ... and, through the barrier, ordered before the ticket
    drew_last = atomicAdd(&tickets[r * nkv + g], 1) == splits - 1;
    if (drew_last) __threadfence();                  // the others' partials, before this block's loads
  }
  __syncthreads();
  if (!drew_last) return;
  // Three rounds of loads instead of a chain: the splits' (max, sum) pairs go to shared memory
  // in one coalesced sweep, each row's weights 2^(m_split - M) are worked out there, and the
  // partial outputs are then read with independent loads.  The sums run in split order.
  const long long base = (((long long)r * nkv + g) * splits) * 16;
  float* ml_s = reinterpret_cast<float*>(smem_raw);      // [splits][16][2]; the tiles' memory is free
  float* w_s = ml_s + splits * 32;                       // [splits][16]
  float* L_s = w_s + splits * 16;                        // [16]
  for (int i = threadIdx.x; i < splits * 32; i += THREADS) ml_s[i] = __ldcg(&part_ml[base * 2 + i]);
  __syncthreads();
  for (int row = threadIdx.x; row < rep; row += THREADS) {
    float M = -INFINITY;
    for (int sp = 0; sp < splits; ++sp) M = fmaxf(M, ml_s[(sp * 16 + row) * 2]);
    const float Mu = M == -INFINITY ? 0.f : M;
    float L = 0.f;
    for (int sp = 0; sp < splits; ++sp) {
      const float f = exp2f(ml_s[(sp * 16 + row) * 2] - Mu);
      w_s[sp * 16 + row] = f;
      L += f * ml_s[(sp * 16 + row) * 2 + 1];
    }
    L_s[row] = L;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rep * HD; idx += THREADS) {
    const int row = idx / HD, d = idx - row * HD;
    const float* po = part_o + (base + row) * HD + d;
    float acc = 0.f;
#pragma unroll 8
    for (int sp = 0; sp < splits; ++sp) acc += w_s[sp * 16 + row] * __ldcg(po + (long long)sp * 16 * HD);
    const float L = L_s[row];
    out[((long long)t * nh + g * rep + row) * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
  }
  if (threadIdx.x == 0) tickets[r * nkv + g] = 0;      // ready for the next launch
}

__global__ void attn_combine_kernel(const float* part_o, const float* part_ml, const int* row_start, bf16* out,
                                    int nh, int nkv, int splits) {
  const int h = blockIdx.x, r = blockIdx.y;
  const int rep = nh / nkv, g = h / rep, row = h - g * rep;
  pdl_wait();
  pdl_trigger();
  const int t = row_start[r];
  const long long base = (((long long)r * nkv + g) * splits) * 16 + row;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[(base + (long long)s * 16) * 2]);
  const float Mu = M == -INFINITY ? 0.f : M;
  float L = 0.f;
  for (int s = 0; s < splits; ++s) {
    const long long pi = base + (long long)s * 16;
    L += exp2f(part_ml[pi * 2] - Mu) * part_ml[pi * 2 + 1];
  }
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      const long long pi = base + (long long)s * 16;
      acc += exp2f(part_ml[pi * 2] - Mu) * part_o[pi * HD + d];
    }
    out[((long long)t * nh + h) * HD + d] = __float2bfloat16_rn(acc * inv);
  }
}

constexpr size_t prefill_smem() { return (size_t)PREFILL_STAGES * 2 * TILE * sizeof(bf16); }
constexpr size_t decode_smem(int kg = 1) {
  const size_t pipe = (size_t)DECODE_STAGES * 2 * 4 * 16 * kg * ROW * sizeof(bf16);
  const size_t merge = (size_t)(4 * 16 * MO_ROW + 4 * 16 * 2 + 16 * HD + 16 * 2) * sizeof(float);
  return pipe > merge ? pipe : merge;
}
// Blocks of the larger tile that an SM holds; the grids that are resident at once with it take it.  (The unsplit
// rows of a large batch do not: alone the kernel was faster with it, batch 64 over 8,192 keys at head size 64 in 174 us
// against 188, but its 512 blocks then take two rounds, and inside a decode step, where no launch of the same kernel
// follows to fill the second round's gaps, the step was 3 to 5 % slower.)
constexpr long long few_per_sm() { return FEW_KG > 1 ? (226 * 1024) / (long long)decode_smem(FEW_KG) : 0; }
bool decode_few(dim3 grid) {
  return FEW_KG > 1 && (long long)grid.x * grid.y * grid.z <= few_per_sm() * fmx_num_sms();
}
template <int NH, int KG> cudaError_t configure_decode_one() {
  cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<DECODE_STAGES, NH, KG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)decode_smem(KG));
  return e;
}
// Can the `splits` blocks of a (row, kv head) run as one cluster?  Asked of the runtime once per size and kernel.
bool g_clusters_allowed = true;
template <int NH, int KG> bool cluster_fits(int splits, dim3 grid) {
  static int known[MAX_CLUSTER + 1];                 // 0: not asked yet, 1: yes, 2: no
  if (!g_clusters_allowed || splits < 2 || splits > MAX_CLUSTER) return false;
  if (known[splits] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = decode_smem(KG);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    const cudaError_t e = cudaOccupancyMaxActiveClusters(&n, attn_decode_kernel<DECODE_STAGES, NH, KG>, &cfg);
    if (e != cudaSuccess) cudaGetLastError();
    known[splits] = (e == cudaSuccess && n > 0) ? 1 : 2;
  }
  return known[splits] == 1;
}
cudaError_t configure_decode() {
  cudaError_t e = configure_decode_one<1, 1>();
  if (e == cudaSuccess) e = configure_decode_one<2, 1>();
  if (e == cudaSuccess && FEW_KG > 1) e = configure_decode_one<1, FEW_KG>();
  if (e == cudaSuccess && FEW_KG > 1) e = configure_decode_one<2, FEW_KG>();
  return e;
}
// The instantiation for a grid and a number of query heads per kv head: LAUNCH(head groups of 8, key groups of 16).
#define FMX_DECODE_DISPATCH(grid, rep, LAUNCH)            \
  do {                                                    \
    if (decode_few(grid)) {                               \
      if ((rep) <= 8) { LAUNCH(1, FEW_KG); } else { LAUNCH(2, FEW_KG); }  \
    } else {                                              \
      if ((rep) <= 8) { LAUNCH(1, 1); } else { LAUNCH(2, 1); }            \
    }                                                     \
  } while (0)
}  // namespace

FMX_EXPORT int fmx_attn_head_dim() { return HD; }

// 0: the splits of a row always combine through L2 and tickets, as they do where a cluster does not fit (for tests
// and timings of that path); 1, the default: through a cluster's shared memory where one fits.  -> the old setting
FMX_EXPORT int fmx_attn_decode_allow_clusters(int allow) {
  const int old = g_clusters_allowed ? 1 : 0;
  g_clusters_allowed = allow != 0;
  return old;
}

// Floats of scratch the decode entry needs for (rows, nkv, splits): partial outputs, then
// their maxima and sums.
FMX_EXPORT long long fmx_attn_decode_scratch_floats(int rows, int nkv, int splits) {
  return splits <= 1 ? 0 : (long long)rows * nkv * splits * 16 * (HD + 2);
}

// How many splits over the keys a decode step of `rows` rows takes on a device of `sms`
// multiprocessors: as many as keep the whole grid resident at once (a second, partial round of
// blocks costs more than it brings), with at least 128 keys to a split and at most 32 splits
// (measured at batch 1 over 8192 keys: 17 to 32 splits 13.5 us, 48: 15.3, 64: 17.7; over 1024
// keys: 2 splits 10.8 us, 8: 6.5).  Up to 32 (row, kv head) pairs the grid is sized for the blocks of the larger
// tile, which the launch then takes (batch 4 over 8192 keys at head size 64: 17.5 us against 18.7).
FMX_EXPORT int fmx_attn_decode_plan(int rows, int nkv, long long max_ctx, int sms) {
  if (sms <= 0) sms = fmx_num_sms();
  const long long pairs = (long long)rows * nkv > 0 ? (long long)rows * nkv : 1;
  long long per_sm = (227 * 1024) / (long long)decode_smem();
  per_sm = per_sm < 1 ? 1 : per_sm > 5 ? 5 : per_sm;
  if (FEW_KG > 1 && pairs <= 32) per_sm = few_per_sm();
  long long s = sms * per_sm / pairs;
  const long long by_keys = (max_ctx + 127) / 128;
  if (s > by_keys) s = by_keys;
  if (s > 32) s = 32;
  // up to 8 splits are one cluster and combine in shared memory, which is worth more than a ninth split (batch 8 over
  // 8,192 keys at head size 64: 8 splits 26.4 us, 9 through tickets 28.9)
  if (s > MAX_CLUSTER && s < 2 * MAX_CLUSTER) s = MAX_CLUSTER;
  return s < 1 ? 1 : (int)s;
}

FMX_EXPORT int fmx_attn_prefill(const void* q, long long q_stride, const void* kv, const int* block_tables,
                                int bt_stride, const int* row_start, const int* row_ctx, void* out, int rows,
                                int max_q_len, int nh, int nkv, int page_size, long long num_pages, float scale,
                                int window, int* status, cudaStream_t stream) {
  if (rows == 0 || max_q_len == 0) return 0;
  if (rows < 0 || nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0)
    return fmx_fail("fmx_attn_prefill: bad sizes rows=%d nh=%d nkv=%d page=%d", rows, nh, nkv, page_size);
  if (rows > 65535 || nkv > 65535) return fmx_fail("fmx_attn_prefill: too many rows or kv heads for one launch");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)prefill_smem());
    if (e != cudaSuccess) return fmx_fail("fmx_attn_prefill: shared memory of %zu bytes refused: %s", prefill_smem(),
                                          cudaGetErrorString(e));
    configured = true;
  }
  const int rep = nh / nkv;
  const long long tiles = ((long long)max_q_len * rep + BM - 1) / BM;
  if (tiles > 65535) return fmx_fail("fmx_attn_prefill: %d query tokens in one row are too many for one launch", max_q_len);
  dim3 grid(nkv, rows, (unsigned)tiles);
  attn_prefill_kernel<<<grid, THREADS, prefill_smem(), stream>>>(
      (const bf16*)q, q_stride, (const bf16*)kv, block_tables, bt_stride, row_start, row_ctx, (bf16*)out, nh, nkv,
      page_size, num_pages, scale, window, status);
  FMX_LAUNCH_CHECK();
  return 0;
}

// tickets: rows * nkv ints, zero before the first call (every call leaves them zero); with
// tickets the last block of each (row, kv head) combines the splits itself, without them a
// second kernel does.  Calls that share scratch or tickets must not overlap on the GPU.
FMX_EXPORT int fmx_attn_decode(const void* q, long long q_stride, const void* kv, const int* block_tables,
                               int bt_stride, const int* row_start, const int* positions, void* out, float* scratch,
                               long long scratch_floats, int* tickets, int rows, int splits, int nh, int nkv,
                               int page_size, long long num_pages, float scale, int window, int* status,
                               const float* inv_freq, int rot, int interleaved, int rope_mode, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rope_mode < 0 || rope_mode > 2 || (rope_mode > 0 && (rot < 0 || rot > HD || (rot & 1) || (rot > 0 && inv_freq == nullptr))))
    return fmx_fail("fmx_attn_decode: bad rotary arguments mode=%d rot=%d", rope_mode, rot);
  if (rows < 0 || nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || splits <= 0)
    return fmx_fail("fmx_attn_decode: bad sizes rows=%d nh=%d nkv=%d page=%d splits=%d", rows, nh, nkv, page_size, splits);
  if (nh / nkv > 16) return fmx_fail("fmx_attn_decode: %d query heads per kv head is above 16", nh / nkv);
  if (splits > 64) return fmx_fail("fmx_attn_decode: at most 64 splits (the combining block stages their statistics in shared memory), not %d", splits);
  if (rows > 65535 || nkv > 65535) return fmx_fail("fmx_attn_decode: too many rows or kv heads for one launch");
  const long long need = fmx_attn_decode_scratch_floats(rows, nkv, splits);
  if (need > 0 && (scratch == nullptr || scratch_floats < need))
    return fmx_fail("fmx_attn_decode: scratch of %lld floats given, %lld needed", scratch_floats, need);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = configure_decode();
    if (e != cudaSuccess) return fmx_fail("fmx_attn_decode: shared memory of %zu bytes refused: %s",
                                          decode_smem(FEW_KG), cudaGetErrorString(e));
    configured = true;
  }
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + (long long)rows * nkv * splits * 16 * HD : nullptr;
  dim3 grid(splits, nkv, rows);
  // With tickets (the engine's calls) and few enough splits, the splits of a row are one cluster and combine through
  // distributed shared memory: no partial goes through L2.
#define FMX_DECODE_LAUNCH(NHG, KGR)                                                                                    \
  do {                                                                                                                  \
    if (tickets != nullptr && cluster_fits<NHG, KGR>(splits, grid))                                                     \
      fmx_launch_cluster(attn_decode_kernel<DECODE_STAGES, NHG, KGR>, grid, dim3(THREADS), decode_smem(KGR), stream,    \
                         dim3(splits, 1, 1), (const bf16*)q, q_stride, (const bf16*)kv, block_tables, bt_stride,        \
                         row_start, positions, (bf16*)out, part_o, part_ml, nh, nkv, page_size, num_pages, scale,       \
                         window, status, tickets, inv_freq, rot, interleaved, rope_mode, 1);                            \
    else                                                                                                                \
      fmx_launch(attn_decode_kernel<DECODE_STAGES, NHG, KGR>, grid, dim3(THREADS), decode_smem(KGR), stream,            \
                 (const bf16*)q, q_stride, (const bf16*)kv, block_tables, bt_stride, row_start, positions, (bf16*)out,  \
                 part_o, part_ml, nh, nkv, page_size, num_pages, scale, window, status, tickets, inv_freq, rot,         \
                 interleaved, rope_mode, 0);                                                                            \
  } while (0)
  FMX_DECODE_DISPATCH(grid, nh / nkv, FMX_DECODE_LAUNCH);
#undef FMX_DECODE_LAUNCH
  FMX_LAUNCH_CHECK();
  if (splits > 1 && tickets == nullptr) {
    fmx_launch(attn_combine_kernel, dim3(nh, rows), dim3(HD < 128 ? 64 : 128), 0, stream, (const float*)part_o,
               (const float*)part_ml, row_start, (bf16*)out, nh, nkv, splits);
    FMX_LAUNCH_CHECK();
  }
  return 0;
}

// ------------------------------------------------------------------------------------
// The same decode attention for callers that cannot allocate: the workspace is a fixed
// array of this module.  See attention_noalloc.h for the contract.
#include "attention_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[FMX_ATTN_NOALLOC_MAX_FLOATS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
// In host code the array's name stands for the symbol, not for a device address: a kernel
// must be given what cudaGetSymbolAddress returns for the current device.
float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};
std::mutex g_noalloc_mutex;          // two threads may make a device's first call at once

int noalloc_setup(float** ptr, cudaStream_t stream) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fmx_fail("fmx_attn_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return fmx_fail("fmx_attn_decode_noalloc: device %d is out of range", dev);
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    // the set-up asks the runtime for an address and an attribute: not inside a stream capture
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    e = cudaStreamIsCapturing(stream, &cap);
    if (e != cudaSuccess) return fmx_fail("fmx_attn_decode_noalloc: cudaStreamIsCapturing: %s", cudaGetErrorString(e));
    if (cap != cudaStreamCaptureStatusNone)
      return fmx_fail("fmx_attn_decode_noalloc: the first call on device %d does its set-up and must come before any "
                      "stream capture; call it once on this device outside the capture", dev);
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fmx_fail("fmx_attn_decode_noalloc: cudaGetSymbolAddress on device %d: %s", dev, cudaGetErrorString(e));
    e = configure_decode();
    if (e != cudaSuccess)
      return fmx_fail("fmx_attn_decode_noalloc: shared memory of %zu bytes refused: %s", decode_smem(FEW_KG),
                      cudaGetErrorString(e));
    g_noalloc_ptr[dev] = p;
  }
  *ptr = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

FMX_EXPORT long long fmx_attn_decode_noalloc_floats(int rows, int nkv, int splits) {
  return splits <= 1 ? 0 : (long long)rows * nkv * splits * 16 * (HD + 2);
}

FMX_EXPORT long long fmx_attn_decode_noalloc_max_floats(void) { return FMX_ATTN_NOALLOC_MAX_FLOATS; }

FMX_EXPORT int fmx_attn_decode_noalloc(const void* q, long long q_stride, const void* kv, const int* block_tables,
                                       int bt_stride, const int* row_start, const int* positions, void* out, int rows,
                                       int splits, int nh, int nkv, int page_size, long long num_pages, float scale,
                                       int window, int* status, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rows < 0 || nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || splits <= 0)
    return fmx_fail("fmx_attn_decode_noalloc: bad sizes rows=%d nh=%d nkv=%d page=%d splits=%d", rows, nh, nkv,
                    page_size, splits);
  if (nh / nkv > 16) return fmx_fail("fmx_attn_decode_noalloc: %d query heads per kv head is above 16", nh / nkv);
  if (rows > 65535 || nkv > 65535) return fmx_fail("fmx_attn_decode_noalloc: too many rows or kv heads for one launch");
  const long long need = fmx_attn_decode_noalloc_floats(rows, nkv, splits);
  if (need > FMX_ATTN_NOALLOC_MAX_FLOATS)
    return fmx_fail("fmx_attn_decode_noalloc: rows=%d nkv=%d splits=%d head_dim=%d need %lld floats of workspace, the "
                    "built-in array holds %d; use fewer splits or fmx_attn_decode with a workspace of your own",
                    rows, nkv, splits, HD, need, FMX_ATTN_NOALLOC_MAX_FLOATS);
  float* scratch = nullptr;
  if (noalloc_setup(&scratch, stream) != 0) return 1;
  float* part_o = scratch;
  float* part_ml = scratch + (long long)rows * nkv * splits * 16 * HD;
  dim3 grid(splits, nkv, rows);
#define FMX_DECODE_LAUNCH(NHG, KGR)                                                                                    \
  attn_decode_kernel<DECODE_STAGES, NHG, KGR><<<grid, THREADS, decode_smem(KGR), stream>>>(                                              \
      (const bf16*)q, q_stride, (const bf16*)kv, block_tables, bt_stride, row_start, positions, (bf16*)out, part_o,     \
      part_ml, nh, nkv, page_size, num_pages, scale, window, status, (int*)nullptr, (const float*)nullptr, 0, 0, 0, 0)
  FMX_DECODE_DISPATCH(grid, nh / nkv, FMX_DECODE_LAUNCH);
#undef FMX_DECODE_LAUNCH
  FMX_LAUNCH_CHECK();
  if (splits > 1) {
    attn_combine_kernel<<<dim3(nh, rows), HD < 128 ? 64 : 128, 0, stream>>>(part_o, part_ml, row_start, (bf16*)out, nh,
                                                                           nkv, splits);
    FMX_LAUNCH_CHECK();
  }
  return 0;
}
