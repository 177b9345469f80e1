// Sampling filters and logits processors on the device, one block per row.
//
// Filters follow tamnd/fastmlx compute/sampler.go:41-173: on the row's log-probabilities,
// in the order top-p, min-p, top-k, each masking tokens out.  The result here is a keep
// mask of one byte per token, which the sampling kernel honours.
//   top-p (0 < p < 1): with tokens ordered by ascending logit (equal logits by ascending
//     index), keep a token when the probability mass up to and including it exceeds 1 - p.
//   min-p (0 < m <= 1): drop tokens whose logit is below max + ln(m) (compared in double),
//     but never the `min_keep` highest (equal logits: lower index first) when min_keep > 1.
//   top-k (0 < k < V): keep the k highest of what is left (equal logits: lower index first).
// No sort is needed: the threshold value of each filter is found by bisection over the
// bit patterns of the floats (32 counting passes), and tokens equal to the threshold are
// told apart by a prefix count in index order.
//
// Processors follow compute/logits_processor.go:61-164, in its order: logit_bias, then the
// repetition penalty (sign-aware, once per distinct token of the window), the presence
// penalty (once per distinct token) and the frequency penalty (per occurrence).
#include <math.h>
#include "common.cuh"

namespace {
constexpr int FBLOCK = 1024;

__device__ __forceinline__ unsigned ordered_key(float f) {
  const unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ float fblock_sum(float v) {
  __shared__ float part[FBLOCK / 32];
  __shared__ float total;
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float s = part[threadIdx.x];
    s = warp_sum(s);
    if (threadIdx.x == 0) total = s;
  }
  __syncthreads();
  const float r = total;
  __syncthreads();
  return r;
}

__device__ float fblock_max(float v) {
  __shared__ float part[FBLOCK / 32];
  __shared__ float total;
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float s = part[threadIdx.x];
    s = warp_max(s);
    if (threadIdx.x == 0) total = s;
  }
  __syncthreads();
  const float r = total;
  __syncthreads();
  return r;
}

// Exclusive prefix over the block in thread order, and the block total.
__device__ float fblock_exscan(float v, float* total) {
  __shared__ float wsum[FBLOCK / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  if (lane == 31) wsum[warp] = x;
  __syncthreads();
  if (warp == 0) {
    float s = wsum[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float y = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += y;
    }
    wsum[lane] = s;
  }
  __syncthreads();
  const float before = warp > 0 ? wsum[warp - 1] : 0.f;
  *total = wsum[FBLOCK / 32 - 1];
  __syncthreads();
  return x - v + before;
}

// Marks in flags[] (bit `bit`) the k highest tokens among those whose keep byte has bit 0
// set (all others count as -inf); equal values: lower index first.  Thread-contiguous
// chunks keep index order across the block.
__device__ void mark_top_k(const float* row, unsigned char* flags, int V, int k, unsigned char bit) {
  const int per = (V + FBLOCK - 1) / FBLOCK;
  const int lo = threadIdx.x * per, hi = min(V, lo + per);
  // largest key x with count(key >= x) >= k
  unsigned xlo = 0u, xhi = 0xffffffffu;
  while (xlo < xhi) {
    const unsigned mid = xlo + (unsigned)(((unsigned long long)xhi - xlo + 1ull) >> 1);
    float cnt = 0.f;
    for (int i = lo; i < hi; ++i) {
      const unsigned key = (flags[i] & 1) ? ordered_key(row[i]) : 0u;
      cnt += key >= mid ? 1.f : 0.f;
    }
    cnt = fblock_sum(cnt);
    if (cnt >= (float)k) xlo = mid; else xhi = mid - 1;
  }
  const unsigned thr = xlo;
  float greater = 0.f, ties = 0.f;
  for (int i = lo; i < hi; ++i) {
    const unsigned key = (flags[i] & 1) ? ordered_key(row[i]) : 0u;
    greater += key > thr ? 1.f : 0.f;
    ties += key == thr ? 1.f : 0.f;
  }
  const float all_greater = fblock_sum(greater);
  float total_ties;
  float rank = fblock_exscan(ties, &total_ties);
  const float room = (float)k - all_greater;
  for (int i = lo; i < hi; ++i) {
    const unsigned key = (flags[i] & 1) ? ordered_key(row[i]) : 0u;
    bool in = key > thr;
    if (key == thr) { in = rank < room; rank += 1.f; }
    if (in) flags[i] |= bit; else flags[i] &= (unsigned char)~bit;
  }
  __syncthreads();
}

__global__ void __launch_bounds__(FBLOCK)
filter_mask_kernel(const float* __restrict__ logits, long long ld, int V, const float* __restrict__ top_p,
                   const float* __restrict__ min_p, const int* __restrict__ top_k, const int* __restrict__ min_keep,
                   unsigned char* __restrict__ keep, long long keep_ld) {
  const int r = blockIdx.x;
  const float* row = logits + (long long)r * ld;
  unsigned char* flags = keep + (long long)r * keep_ld;
  const int per = (V + FBLOCK - 1) / FBLOCK;
  const int lo = threadIdx.x * per, hi = min(V, lo + per);
  for (int i = lo; i < hi; ++i) flags[i] = 1;
  __syncthreads();

  float mx = -INFINITY;
  for (int i = lo; i < hi; ++i) mx = fmaxf(mx, row[i]);
  mx = fblock_max(mx);

  const float p = top_p ? top_p[r] : 0.f;
  if (p > 0.f && p < 1.f) {
    float z = 0.f;
    for (int i = lo; i < hi; ++i) z += expf(row[i] - mx);
    z = fblock_sum(z);
    const float need = (1.0f - p) * z;              // keep when the ascending mass exceeds this
    // smallest key x with mass(key <= x) > need
    unsigned xlo = 0u, xhi = 0xffffffffu;
    while (xlo < xhi) {
      const unsigned mid = xlo + ((xhi - xlo) >> 1);
      float s = 0.f;
      for (int i = lo; i < hi; ++i) s += ordered_key(row[i]) <= mid ? expf(row[i] - mx) : 0.f;
      s = fblock_sum(s);
      if (s > need) xhi = mid; else xlo = mid + 1;
    }
    const unsigned thr = xlo;
    float below = 0.f, tie = 0.f;
    for (int i = lo; i < hi; ++i) {
      const unsigned key = ordered_key(row[i]);
      const float w = expf(row[i] - mx);
      below += key < thr ? w : 0.f;
      tie += key == thr ? w : 0.f;
    }
    const float all_below = fblock_sum(below);
    float tie_total;
    float run = all_below + fblock_exscan(tie, &tie_total);
    for (int i = lo; i < hi; ++i) {
      const unsigned key = ordered_key(row[i]);
      bool in = key > thr;
      if (key == thr) { run += expf(row[i] - mx); in = run > need; }
      flags[i] = in ? 1 : 0;
    }
    __syncthreads();
  }

  const float m = min_p ? min_p[r] : 0.f;
  if (m > 0.f && m <= 1.f) {
    const int mk = min_keep ? min_keep[r] : 0;
    if (mk > 1) mark_top_k(row, flags, V, mk, 2);
    const double floor_ = (double)mx + log((double)m);
    for (int i = lo; i < hi; ++i) {
      if (!(flags[i] & 1)) { flags[i] = 0; continue; }
      const bool drop = (double)row[i] < floor_ && !(flags[i] & 2);
      flags[i] = drop ? 0 : 1;
    }
    __syncthreads();
  }

  const int kk = top_k ? top_k[r] : 0;
  if (kk > 0 && kk < V) {
    mark_top_k(row, flags, V, kk, 4);
    for (int i = lo; i < hi; ++i) flags[i] = ((flags[i] & 1) && (flags[i] & 4)) ? 1 : 0;
    __syncthreads();
  }
}

// One block per row; history[r, :] holds the row's last tokens (oldest first), -1 padded
// at the front.  Each penalty looks at its own trailing window of the history.
__global__ void penalties_kernel(float* __restrict__ logits, long long ld, int V, const int* __restrict__ history,
                                 int H, const float* __restrict__ repetition, const float* __restrict__ presence,
                                 const float* __restrict__ frequency, const int* __restrict__ windows) {
  const int r = blockIdx.x;
  float* row = logits + (long long)r * ld;
  const int* hist = history + (long long)r * H;
  const float rep = repetition ? repetition[r] : 1.f;
  const float pres = presence ? presence[r] : 0.f;
  const float freq = frequency ? frequency[r] : 0.f;
  const int wrep = windows[r * 3 + 0], wpres = windows[r * 3 + 1], wfreq = windows[r * 3 + 2];
  // Phase by phase, so that a later penalty sees what the earlier one wrote.
  for (int phase = 0; phase < 3; ++phase) {
    const int w = phase == 0 ? wrep : phase == 1 ? wpres : wfreq;
    const bool on = phase == 0 ? (rep != 1.f && rep != 0.f) : phase == 1 ? (pres != 0.f) : (freq != 0.f);
    if (on) {
      const int start = max(0, H - w);
      for (int i = start + threadIdx.x; i < H; i += blockDim.x) {
        const int t = hist[i];
        if (t < 0 || t >= V) continue;
        int count = 0;
        bool first = true;
        for (int j = start; j < H; ++j) {
          if (hist[j] == t) { ++count; if (j < i) first = false; }
        }
        if (!first) continue;                        // one thread per distinct token
        float v = row[t];
        if (phase == 0) v = v < 0.f ? v * rep : v / rep;
        else if (phase == 1) v -= pres;
        else for (int c = 0; c < count; ++c) v -= freq;      // per occurrence, one subtraction each
        row[t] = v;
      }
    }
    __syncthreads();
  }
}

__global__ void logit_bias_kernel(float* __restrict__ logits, long long ld, int V, const int* __restrict__ rows,
                                  const int* __restrict__ ids, const float* __restrict__ values, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int id = ids[i];
  if (id < 0 || id >= V) return;
  atomicAdd(&logits[(long long)rows[i] * ld + id], values[i]);
}
}  // namespace

FMX_EXPORT int fmx_filter_mask(const float* logits, long long ld, int rows, int V, const float* top_p,
                               const float* min_p, const int* top_k, const int* min_keep, unsigned char* keep,
                               long long keep_ld, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rows < 0 || V <= 0 || ld < V || keep_ld < V) return fmx_fail("fmx_filter_mask: bad sizes rows=%d V=%d", rows, V);
  if (V > (1 << 24)) return fmx_fail("fmx_filter_mask: a vocabulary of %d is beyond exact float counting", V);
  filter_mask_kernel<<<rows, FBLOCK, 0, stream>>>(logits, ld, V, top_p, min_p, top_k, min_keep, keep, keep_ld);
  FMX_LAUNCH_CHECK();
  return 0;
}

FMX_EXPORT int fmx_penalties(float* logits, long long ld, int rows, int V, const int* history, int H,
                             const float* repetition, const float* presence, const float* frequency,
                             const int* windows, cudaStream_t stream) {
  if (rows == 0 || H == 0) return 0;
  if (rows < 0 || V <= 0 || H < 0) return fmx_fail("fmx_penalties: bad sizes rows=%d V=%d H=%d", rows, V, H);
  penalties_kernel<<<rows, 128, 0, stream>>>(logits, ld, V, history, H, repetition, presence, frequency, windows);
  FMX_LAUNCH_CHECK();
  return 0;
}

FMX_EXPORT int fmx_logit_bias(float* logits, long long ld, int V, const int* rows, const int* ids, const float* values,
                              int n, cudaStream_t stream) {
  if (n == 0) return 0;
  logit_bias_kernel<<<(n + 127) / 128, 128, 0, stream>>>(logits, ld, V, rows, ids, values, n);
  FMX_LAUNCH_CHECK();
  return 0;
}
