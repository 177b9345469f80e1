// Greedy choice and temperature sampling over 32-bit logits, one block per row.
//
// tamnd/fastmlx takes argmax at temperature 0, the first index on ties
// (compute/sampler.go:38-39,61-72), and otherwise draws from softmax(logits / T) after its
// filters; the draw itself is left to the tensor library there (sampler.go:17-22).  Here
// the draw is an inverse-CDF walk in index order with a uniform number that the caller
// derives from (seed, request, token index), so the token does not depend on what else is
// in the batch.  Filters (top-p, min-p, top-k) are applied by the caller as a keep mask of
// one byte per token, or none.
#include <math.h>
#include "common.cuh"

namespace {
constexpr int SBLOCK = 1024;

struct Best { float v; int i; };

__device__ __forceinline__ Best better(Best a, Best b) {
  // higher value wins; on equal values the lower index
  if (b.i >= 0 && (a.i < 0 || b.v > a.v || (b.v == a.v && b.i < a.i))) return b;
  return a;
}

__device__ Best block_argmax(const float* row, const unsigned char* keep, int V) {
  __shared__ Best part[SBLOCK / 32];
  __shared__ Best result;
  Best b{-INFINITY, -1};
  int done = 0;
  if (keep == nullptr && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    // four logits per load, several loads in flight; a thread meets its indices in rising order
    const int V4 = V / 4;
    const float4* row4 = reinterpret_cast<const float4*>(row);
#pragma unroll 4
    for (int i = threadIdx.x; i < V4; i += SBLOCK) {
      const float4 v = row4[i];
      const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (b.i < 0 || e[j] > b.v) b = Best{e[j], 4 * i + j};
    }
    done = 4 * V4;
  }
  for (int i = done + threadIdx.x; i < V; i += SBLOCK) {
    if (keep && !keep[i]) continue;
    const float v = row[i];
    if (b.i < 0 || v > b.v) b = Best{v, i};
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
    b = better(b, other);
  }
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = b;
  __syncthreads();
  if (threadIdx.x < 32) {
    Best c = threadIdx.x < SBLOCK / 32 ? part[threadIdx.x] : Best{-INFINITY, -1};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best other{__shfl_xor_sync(0xffffffffu, c.v, o), __shfl_xor_sync(0xffffffffu, c.i, o)};
      c = better(c, other);
    }
    if (threadIdx.x == 0) result = c;
  }
  __syncthreads();
  Best r = result;
  __syncthreads();
  return r;
}

// Greedy choice with a row cut into chunks, one block each: at a vocabulary of 10^5 a single block
// per row spends 15 us reading its half megabyte while most SMs idle.  A block leaves its
// chunk's best in `partial` and takes a ticket; the row's last block compares the chunks' bests in
// chunk order (ties still go to the lower index) and sets the ticket back to zero.
constexpr int ABLOCK = 256;

__global__ void __launch_bounds__(ABLOCK)
argmax_split_kernel(const float* logits, long long ld, int V, int chunk, Best* partial, int* tickets, int* out) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.y, c = blockIdx.x, chunks = gridDim.x;
  const float* row = logits + (long long)r * ld;
  const int lo = c * chunk, hi = min(V, lo + chunk);       // chunk is a multiple of 4
  Best b{-INFINITY, -1};
  int done = lo;
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int lo4 = lo / 4, hi4 = hi / 4;
#pragma unroll 4
    for (int i = lo4 + threadIdx.x; i < hi4; i += ABLOCK) {
      const float4 v = row4[i];
      const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (b.i < 0 || e[j] > b.v) b = Best{e[j], 4 * i + j};
    }
    done = max(lo, 4 * hi4);
  }
  for (int i = done + threadIdx.x; i < hi; i += ABLOCK) {
    const float v = row[i];
    if (b.i < 0 || v > b.v) b = Best{v, i};
  }
  __shared__ Best part[ABLOCK / 32];
  __shared__ bool last;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
    b = better(b, other);
  }
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = b;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < ABLOCK / 32; ++w) b = better(b, part[w]);
    partial[(long long)r * chunks + c] = b;
    __threadfence();
    last = atomicAdd(&tickets[r], 1) == chunks - 1;
  }
  __syncthreads();
  if (!last || threadIdx.x >= 32) return;
  __threadfence();
  Best t{-INFINITY, -1};
  for (int j = threadIdx.x; j < chunks; j += 32) {
    const volatile Best* p = partial + (long long)r * chunks + j;
    t = better(t, Best{p->v, p->i});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
    t = better(t, other);
  }
  if (threadIdx.x == 0) {
    out[r] = t.i;
    tickets[r] = 0;
  }
}

// Inclusive prefix sum over the block in thread order; returns this thread's inclusive
// value and the block total.
__device__ float block_scan(float v, float* total) {
  __shared__ float wsum[SBLOCK / 32];
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
  *total = wsum[SBLOCK / 32 - 1];
  __syncthreads();
  return x + before;
}

__global__ void __launch_bounds__(SBLOCK)
sample_kernel(const float* logits, long long ld, int V, const float* temperature, const float* uniform,
              const unsigned char* keep, long long keep_ld, int* out) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const float* row = logits + (long long)r * ld;
  const unsigned char* kp = keep ? keep + (long long)r * keep_ld : nullptr;
  const Best top = block_argmax(row, kp, V);
  const float T = temperature ? temperature[r] : 0.f;
  if (!(T > 0.f) || top.i < 0) {
    if (threadIdx.x == 0) out[r] = top.i;
    return;
  }
  const float inv_t = 1.0f / T;
  // total weight, each thread over a contiguous chunk so that the walk below is in index order
  const int per = (V + SBLOCK - 1) / SBLOCK;
  const int lo = threadIdx.x * per, hi = min(V, lo + per);
  float mine = 0.f;
  for (int i = lo; i < hi; ++i)
    if (!kp || kp[i]) mine += expf((row[i] - top.v) * inv_t);
  float total;
  const float incl = block_scan(mine, &total);
  const float target = uniform[r] * total;
  __shared__ int chosen;
  if (threadIdx.x == 0) chosen = -1;
  __syncthreads();
  const float before = incl - mine;
  if (mine > 0.f && target >= before && target < incl) {
    float run = before;
    int pick = -1;
    for (int i = lo; i < hi; ++i) {
      if (kp && !kp[i]) continue;
      const float wgt = expf((row[i] - top.v) * inv_t);
      if (wgt <= 0.f) continue;
      pick = i;
      run += wgt;
      if (target < run) break;
    }
    chosen = pick;
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = chosen >= 0 ? chosen : top.i;   // rounding at the far end: the mode
}
}  // namespace

// out[r] = argmax of row r (first index on ties) where temperature[r] <= 0 or temperature is
// null; else a draw from softmax(row / temperature[r]) restricted to keep[r, :] != 0, by the
// uniform number uniform[r] in [0, 1).
// Greedy rows without a keep mask are cut into `chunks` blocks each when a workspace is given:
// partial holds ticket_rows x partial_chunks pairs (value, index) of 8 bytes, tickets ticket_rows
// ints that are zero between launches.
FMX_EXPORT int fmx_sample(const float* logits, long long ld, int rows, int V, const float* temperature,
                          const float* uniform, const unsigned char* keep, long long keep_ld, int* out,
                          int chunks, void* partial, int partial_chunks, int* tickets, int ticket_rows,
                          cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rows < 0 || V <= 0 || ld < V) return fmx_fail("fmx_sample: bad sizes rows=%d V=%d ld=%lld", rows, V, ld);
  if (temperature != nullptr && uniform == nullptr) return fmx_fail("fmx_sample: a temperature needs uniform numbers");
  if (temperature == nullptr && keep == nullptr && partial != nullptr && chunks > 1) {
    if (chunks > partial_chunks || rows > ticket_rows)
      return fmx_fail("fmx_sample: %d rows in %d chunks do not fit the workspace (%d rows, %d chunks)", rows, chunks,
                      ticket_rows, partial_chunks);
    const int chunk = ((V + chunks - 1) / chunks + 3) / 4 * 4;
    fmx_launch(argmax_split_kernel, dim3((V + chunk - 1) / chunk, rows), dim3(ABLOCK), 0, stream, logits, ld, V, chunk,
               reinterpret_cast<Best*>(partial), tickets, out);
    FMX_LAUNCH_CHECK();
    return 0;
  }
  fmx_launch(sample_kernel, dim3(rows), dim3(SBLOCK), 0, stream, logits, ld, V, temperature, uniform, keep, keep_ld, out);
  FMX_LAUNCH_CHECK();
  return 0;
}
