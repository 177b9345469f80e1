// Paged grouped-query attention, one warp per (query token, query head).
//
// The kernel of the true 32-bit path, and the fallback of the bfloat16 path for head
// sizes its tiled kernels do not take.  A query at position p of row r sees the keys of
// its request at positions lo..p (lo = max(0, p - window + 1) with a window, else 0), all
// read from the pages the row's block table names.  Keys are taken 32 at a time, chunks
// aligned to absolute positions (0-31, 32-63, ...), one key per lane; scores, the running
// maximum and sum, and the output accumulator are 32-bit.  The order of every sum depends
// only on the key's position, never on how the tokens were cut into steps or on what else
// is in the batch.
#include <math.h>
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_HD = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_simple_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ kv,
                              const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ token_row,
                              const int* __restrict__ positions, T* __restrict__ out, int n_tokens, int nh, int nkv,
                              int hd, int page_size, long long num_pages, float scale, int window, int R,
                              int* status) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * WARPS + warp;
  if (w >= (long long)n_tokens * nh) return;
  const int t = (int)(w / nh), h = (int)(w - (long long)t * nh);
  const int g = h / (nh / nkv);
  float* qs = smem + warp * hd;
  const T* qp = q + (long long)t * q_stride + (long long)h * hd;
  for (int e = lane; e < hd; e += 32) qs[e] = to_f(qp[e]);
  __syncwarp();

  const int row = token_row[t];
  T* op = out + ((long long)t * nh + h) * hd;
  if (row < 0 || row >= R) {
    if (lane == 0) fmx_set_status(status, FMX_BAD_ROW, row, t);
    for (int e = lane; e < hd; e += 32) op[e] = from_f<T>(0.f);
    return;
  }
  const int pos = positions[t];
  const int* bt = block_tables + (long long)row * bt_stride;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const long long plane = (long long)nkv * page_size * hd;     // k plane -> v plane of a page

  float m = -INFINITY, l = 0.f;
  float acc[MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) acc[i] = 0.f;

  for (int c = lo / 32; c * 32 <= pos; ++c) {
    const int j = c * 32 + lane;
    bool valid = j >= lo && j <= pos;
    float s = -INFINITY;
    long long vbase = 0;
    if (valid) {
      const int blk = j / page_size;
      const int page = blk < bt_stride ? bt[blk] : -1;
      if (page < 0 || page >= num_pages) {
        fmx_set_status(status, FMX_BAD_PAGE, page, t);
        valid = false;
      } else {
        const long long kbase = ((((long long)page * 2) * nkv + g) * page_size + (j - blk * page_size)) * hd;
        vbase = kbase + plane;
        float dot = 0.f;
        for (int e = 0; e < hd; ++e) dot = fmaf(qs[e], to_f(kv[kbase + e]), dot);
        s = dot * scale;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;
    const float p = valid ? expf(s - m_new) : 0.f;
    const float alpha = expf(m - m_new);
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) acc[i] *= alpha;
    for (int jj = 0; jj < 32; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long vb = __shfl_sync(0xffffffffu, vbase, jj);
      if (pj == 0.f) continue;                // keys out of sight are never read
#pragma unroll
      for (int i = 0; i < MAX_HD / 32; ++i) {
        const int e = lane + 32 * i;
        if (e < hd) acc[i] = fmaf(pj, to_f(kv[vb + e]), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) {
    const int e = lane + 32 * i;
    if (e < hd) op[e] = from_f<T>(acc[i] * inv);
  }
}
}  // namespace

FMX_EXPORT int fmx_paged_attention_simple(const void* q, long long q_stride, const void* kv, const int* block_tables,
                                          int bt_stride, const int* token_row, const int* positions, void* out,
                                          int n_tokens, int nh, int nkv, int hd, int page_size, long long num_pages,
                                          float scale, int window, int R, int dtype, int* status,
                                          cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  if (n_tokens < 0 || nh <= 0 || nkv <= 0 || nh % nkv || hd <= 0 || page_size <= 0)
    return fmx_fail("fmx_paged_attention_simple: bad sizes T=%d nh=%d nkv=%d hd=%d page=%d", n_tokens, nh, nkv, hd,
                    page_size);
  if (hd > MAX_HD) return fmx_fail("fmx_paged_attention_simple: head size %d is above %d", hd, MAX_HD);
  const long long warps = (long long)n_tokens * nh;
  const long long grid = (warps + WARPS - 1) / WARPS;
  if (grid > 2147483647LL) return fmx_fail("fmx_paged_attention_simple: batch too large");
  const size_t smem = (size_t)WARPS * hd * sizeof(float);
  if (dtype == FMX_F32)
    paged_attention_simple_kernel<float><<<(unsigned)grid, WARPS * 32, smem, stream>>>(
        (const float*)q, q_stride, (const float*)kv, block_tables, bt_stride, token_row, positions, (float*)out,
        n_tokens, nh, nkv, hd, page_size, num_pages, scale, window, R, status);
  else if (dtype == FMX_BF16)
    paged_attention_simple_kernel<bf16><<<(unsigned)grid, WARPS * 32, smem, stream>>>(
        (const bf16*)q, q_stride, (const bf16*)kv, block_tables, bt_stride, token_row, positions, (bf16*)out, n_tokens,
        nh, nkv, hd, page_size, num_pages, scale, window, R, status);
  else
    return fmx_fail("fmx_paged_attention_simple: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}
