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

// ------------------------------------------------------------------------------------ a row on a cluster
// The same filters with a row spread over a thread-block cluster of FC blocks of 1024 threads: every thread keeps
// its EPT consecutive logits (as ordered keys and, for top-p, as weights exp(logit - max)) in registers, so that a
// pass of a bisection neither reads memory nor calls expf again; a pass costs one block sum and one exchange of
// the FC blocks' sums through distributed shared memory (summed in rank order by every block: all blocks take the
// same decision from the same bits).  With one block per row a 128,256-wide row took 1.0 ms for top-p alone and
// 2.6 ms for top-p and top-k, on one SM per row.
constexpr int FC = 8;

__device__ __forceinline__ unsigned fc_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void fc_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float fc_peer(const float* local, unsigned rank) {
  unsigned remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((unsigned)__cvta_generic_to_shared(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// Sums (or maxima) over the whole cluster, the same bits in every block.  `slot` alternates between two places so
// that a block may write its next partial while a peer still reads the last one (a peer that has passed the
// barrier of exchange n has finished reading exchange n - 1).
struct FcExchange {
  float* part;      // [4] in shared memory, the same place in every block: two slots of up to two values
  int at;
  float (*warps)[FBLOCK / 32];      // [2][32]: the warps' partials of the block's own sum, two slots as well
  // One block barrier and one cluster barrier per exchange (a bisection makes 32 of them): the warps' sums meet in
  // the first warp, whose first lane leaves the block's sum where the cluster reads it.
  __device__ float sum(float v) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    if (lane == 0) warps[at][warp] = v;
    __syncthreads();
    if (warp == 0) {
      const float s = warp_sum(warps[at][lane]);
      if (lane == 0) part[at] = s;
    }
    fc_sync();
    float s = 0.f;
#pragma unroll
    for (unsigned r = 0; r < FC; ++r) s += fc_peer(part + at, r);
    at ^= 1;
    return s;
  }
  __device__ float max(float v) {
    v = fblock_max(v);
    if (threadIdx.x == 0) part[at] = v;
    fc_sync();
    float s = -INFINITY;
#pragma unroll
    for (unsigned r = 0; r < FC; ++r) s = fmaxf(s, fc_peer(part + at, r));
    at ^= 1;
    return s;
  }
  // two maxima in one exchange
  __device__ void max2(float& a, float& b) {
    a = fblock_max(a);
    b = fblock_max(b);
    if (threadIdx.x == 0) {
      part[at] = a;
      part[2 + at] = b;
    }
    fc_sync();
    a = b = -INFINITY;
#pragma unroll
    for (unsigned r = 0; r < FC; ++r) {
      a = fmaxf(a, fc_peer(part + at, r));
      b = fmaxf(b, fc_peer(part + 2 + at, r));
    }
    at ^= 1;
  }
  // exclusive prefix in index order (rank, then thread); *all: the sum over the whole cluster, in rank order
  __device__ float exscan(float v, float* all = nullptr) {
    float total;
    const float before = fblock_exscan(v, &total);
    if (threadIdx.x == 0) part[at] = total;
    fc_sync();
    float lower = 0.f, whole = 0.f;
    const unsigned me = fc_rank();
#pragma unroll
    for (unsigned r = 0; r < FC; ++r) {
      const float t = fc_peer(part + at, r);
      lower += r < me ? t : 0.f;
      whole += t;
    }
    at ^= 1;
    if (all != nullptr) *all = whole;
    return lower + before;
  }
};

// Marks (bit e of the result) the k highest among this thread's elements that are alive; equal keys: lower index first.
template <int EPT>
__device__ unsigned fc_top_k(const unsigned (&key)[EPT], unsigned alive, int k, FcExchange& x) {
  unsigned xlo = 0u, xhi = 0xffffffffu;
  while (xlo < xhi) {                                 // largest x with count(key >= x) >= k
    const unsigned mid = xlo + (unsigned)(((unsigned long long)xhi - xlo + 1ull) >> 1);
    float cnt = 0.f;
#pragma unroll
    for (int e = 0; e < EPT; ++e) cnt += (((alive >> e) & 1u) ? key[e] : 0u) >= mid ? 1.f : 0.f;
    if (x.sum(cnt) >= (float)k) xlo = mid; else xhi = mid - 1;
  }
  const unsigned thr = xlo;
  float greater = 0.f, ties = 0.f;
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    const unsigned ke = ((alive >> e) & 1u) ? key[e] : 0u;
    greater += ke > thr ? 1.f : 0.f;
    ties += ke == thr ? 1.f : 0.f;
  }
  const float room = (float)k - x.sum(greater);
  float rank = x.exscan(ties);
  unsigned marked = 0u;
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    const unsigned ke = ((alive >> e) & 1u) ? key[e] : 0u;
    bool in = ke > thr;
    if (ke == thr) { in = rank < room; rank += 1.f; }
    marked |= in ? (1u << e) : 0u;
  }
  return marked;
}

template <int EPT>
__global__ void __launch_bounds__(FBLOCK)
filter_mask_cluster_kernel(const float* __restrict__ logits, long long ld, int V, const float* __restrict__ top_p,
                           const float* __restrict__ min_p, const int* __restrict__ top_k,
                           const int* __restrict__ min_keep, unsigned char* __restrict__ keep, long long keep_ld,
                           const float* __restrict__ temperature, const float* __restrict__ uniform, int* __restrict__ out) {
  __shared__ float part[4];
  __shared__ float warps[2][FBLOCK / 32];
  FcExchange x{part, 0, warps};
  const int r = blockIdx.x / FC;
  const unsigned rank = fc_rank();
  const float* row = logits + (long long)r * ld;
  unsigned char* flags = keep ? keep + (long long)r * keep_ld : nullptr;
  const int base = ((int)rank * FBLOCK + threadIdx.x) * EPT;      // thread-contiguous: index order is (rank, thread, e)
  float val[EPT];
  unsigned key[EPT];
  unsigned alive = 0u;
  float mx = -INFINITY;
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    const bool in = base + e < V;
    val[e] = in ? row[base + e] : -INFINITY;
    key[e] = in ? ordered_key(val[e]) : 0u;
    alive |= in ? (1u << e) : 0u;
    mx = fmaxf(mx, val[e]);
  }
  const unsigned valid = alive;
  mx = x.max(mx);

  const float p = top_p ? top_p[r] : 0.f;
  if (p > 0.f && p < 1.f) {
    float w[EPT], z = 0.f;
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
      w[e] = ((valid >> e) & 1u) ? expf(val[e] - mx) : 0.f;
      z += w[e];
    }
    const float need = (1.0f - p) * x.sum(z);          // keep when the ascending mass exceeds this
    unsigned xlo = 0u, xhi = 0xffffffffu;
    while (xlo < xhi) {                                // smallest x with mass(key <= x) > need
      const unsigned mid = xlo + ((xhi - xlo) >> 1);
      float sm = 0.f;
#pragma unroll
      for (int e = 0; e < EPT; ++e) sm += (((valid >> e) & 1u) && key[e] <= mid) ? w[e] : 0.f;
      if (x.sum(sm) > need) xhi = mid; else xlo = mid + 1;
    }
    const unsigned thr = xlo;
    float below = 0.f, tie = 0.f;
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
      const bool on = (valid >> e) & 1u;
      below += (on && key[e] < thr) ? w[e] : 0.f;
      tie += (on && key[e] == thr) ? w[e] : 0.f;
    }
    const float all_below = x.sum(below);
    float run = all_below + x.exscan(tie);
    alive = 0u;
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
      if (!((valid >> e) & 1u)) continue;
      bool in = key[e] > thr;
      if (key[e] == thr) { run += w[e]; in = run > need; }
      alive |= in ? (1u << e) : 0u;
    }
  }

  const float m = min_p ? min_p[r] : 0.f;
  if (m > 0.f && m <= 1.f) {
    const int mk = min_keep ? min_keep[r] : 0;
    const unsigned kept = mk > 1 ? fc_top_k<EPT>(key, alive, mk, x) : 0u;
    const double floor_ = (double)mx + log((double)m);
    unsigned next = 0u;
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
      if (!((alive >> e) & 1u)) continue;
      const bool drop = (double)val[e] < floor_ && !((kept >> e) & 1u);
      next |= drop ? 0u : (1u << e);
    }
    alive = next;
  }

  const int kk = top_k ? top_k[r] : 0;
  if (kk > 0 && kk < V) alive &= fc_top_k<EPT>(key, alive, kk, x);

  if (flags != nullptr) {
#pragma unroll
    for (int e = 0; e < EPT; ++e)
      if ((valid >> e) & 1u) flags[base + e] = (alive >> e) & 1u;
  }
  if (out != nullptr) {
    // The token, as sample_kernel chooses it from a keep mask: the first index of the largest logit at temperature 0
    // (the largest logit is always kept), else the inverse-CDF walk in index order over exp((logit - max) / T).
    const float T = temperature ? temperature[r] : 0.f;
    const float inv_t = T > 0.f ? 1.0f / T : 0.f;
    float cand = -INFINITY, last = -INFINITY;          // minus the first index of the largest logit; the last index with weight
#pragma unroll
    for (int e = EPT - 1; e >= 0; --e)
      if (((alive >> e) & 1u) && val[e] == mx) cand = -(float)(base + e);
#pragma unroll
    for (int e = 0; e < EPT; ++e)
      if (((alive >> e) & 1u) && expf((val[e] - mx) * inv_t) > 0.f) last = (float)(base + e);
    x.max2(cand, last);                                // indices are below 2^24: exact as floats
    // What stands unless a thread below finds the target inside its own share: the mode at temperature 0; else the
    // last token with weight, which is where a target within rounding of the total belongs.
    if (rank == 0 && threadIdx.x == 0) out[r] = T > 0.f && last >= 0.f ? (int)last : (int)(-cand);
    if (T > 0.f) {
      float mine = 0.f;
#pragma unroll
      for (int e = 0; e < EPT; ++e) mine += ((alive >> e) & 1u) ? expf((val[e] - mx) * inv_t) : 0.f;
      float total;
      const float before = x.exscan(mine, &total);     // its barrier also orders the store above before the draw's
      const float target = uniform[r] * total;
      if (mine > 0.f && target >= before && target < before + mine) {
        float run = before;
        int pick = -1;
#pragma unroll
        for (int e = 0; e < EPT; ++e) {
          const float wgt = ((alive >> e) & 1u) ? expf((val[e] - mx) * inv_t) : 0.f;
          if (wgt > 0.f && (pick < 0 || target >= run)) {       // the first element whose running sum passes the target
            pick = base + e;
            run += wgt;
          }
        }
        out[r] = pick;
      }
    }
  }
  fc_sync();                                           // nobody leaves while a peer may still read its sums
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

namespace {
// A wide row goes to a cluster of FC blocks with the row in registers; narrow ones, and rows beyond 131,072 (whose
// share per thread would not fit the registers of a 1024-thread block), to one block.
bool row_fits_a_cluster(int V) { return V > 16384 && (V + FC * FBLOCK - 1) / (FC * FBLOCK) <= 16; }

int launch_cluster_filter(const float* logits, long long ld, int rows, int V, const float* top_p, const float* min_p,
                          const int* top_k, const int* min_keep, unsigned char* keep, long long keep_ld,
                          const float* temperature, const float* uniform, int* out, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)rows * FC);
  cfg.blockDim = dim3(FBLOCK);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = FC;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, filter_mask_cluster_kernel<16>, logits, ld, V, top_p, min_p, top_k, min_keep, keep,
                                     keep_ld, temperature, uniform, out);
  if (e != cudaSuccess) return fmx_fail("the filters' cluster kernel: launch failed: %s", cudaGetErrorString(e));
  FMX_LAUNCH_CHECK();
  return 0;
}
}  // namespace

FMX_EXPORT int fmx_filter_mask(const float* logits, long long ld, int rows, int V, const float* top_p,
                               const float* min_p, const int* top_k, const int* min_keep, unsigned char* keep,
                               long long keep_ld, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rows < 0 || V <= 0 || ld < V || keep_ld < V) return fmx_fail("fmx_filter_mask: bad sizes rows=%d V=%d", rows, V);
  if (V > (1 << 24)) return fmx_fail("fmx_filter_mask: a vocabulary of %d is beyond exact float counting", V);
  if (row_fits_a_cluster(V))
    return launch_cluster_filter(logits, ld, rows, V, top_p, min_p, top_k, min_keep, keep, keep_ld, nullptr, nullptr, nullptr,
                                 stream);
  filter_mask_kernel<<<rows, FBLOCK, 0, stream>>>(logits, ld, V, top_p, min_p, top_k, min_keep, keep, keep_ld);
  FMX_LAUNCH_CHECK();
  return 0;
}

// Can fmx_filter_sample take rows of this width?
FMX_EXPORT int fmx_filter_sample_takes(int V) { return row_fits_a_cluster(V) ? 1 : 0; }

// Filters and the choice of the token in one kernel, no keep mask in memory: out[r] as fmx_sample would choose it
// from the mask that fmx_filter_mask would have written (any filter argument may be null: off).  Rows of the widths
// that fmx_filter_sample_takes only.
FMX_EXPORT int fmx_filter_sample(const float* logits, long long ld, int rows, int V, const float* temperature,
                                 const float* uniform, const float* top_p, const float* min_p, const int* top_k,
                                 const int* min_keep, int* out, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rows < 0 || V <= 0 || ld < V) return fmx_fail("fmx_filter_sample: bad sizes rows=%d V=%d", rows, V);
  if (!row_fits_a_cluster(V)) return fmx_fail("fmx_filter_sample: rows of %d logits go to fmx_filter_mask and fmx_sample", V);
  if (temperature != nullptr && uniform == nullptr) return fmx_fail("fmx_filter_sample: a temperature needs uniform numbers");
  return launch_cluster_filter(logits, ld, rows, V, top_p, min_p, top_k, min_keep, nullptr, 0, temperature, uniform, out, stream);
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
