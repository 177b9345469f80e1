// Rotary positions on q and k, fused with the write of k and v into the layer's pages.
//
// qkv is [T, (nh + 2 nkv) * hd]: nh query heads, nkv key heads, nkv value heads.  q and k
// are rotated in place (angle = position * inv_freq[j] in 32-bit, sine and cosine by the
// accurate sincosf); the rotated k and the v of token t then go to slot_mapping[t] of a
// cache laid out [page, 2 (k|v), nkv, page_size, hd].  With nkv = 0 only q is rotated;
// with rot = 0 nothing is rotated and the kernel only stores.
#include "common.cuh"

template <typename T>
__global__ void rope_kv_write_kernel(T* qkv, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                     const long long* __restrict__ slot_mapping, T* kv, int nh, int nkv, int hd, int rot,
                                     int interleaved, int page_size, long long num_pages, long long row_stride,
                                     int* status) {
  const int t = blockIdx.x;
  T* row = qkv + (long long)t * row_stride;
  const int half = rot / 2;
  if (half > 0) {
    const float pos = (float)positions[t];
    const int items = (nh + nkv) * half;
    for (int it = threadIdx.x; it < items; it += blockDim.x) {
      const int h = it / half, j = it - h * half;
      T* p = row + (long long)h * hd;
      const int i0 = interleaved ? 2 * j : j;
      const int i1 = interleaved ? 2 * j + 1 : j + half;
      const float a = to_f(p[i0]), b = to_f(p[i1]);
      float s, c;
      sincosf(pos * inv_freq[j], &s, &c);
      p[i0] = from_f<T>(a * c - b * s);
      p[i1] = from_f<T>(b * c + a * s);
    }
  }
  if (kv == nullptr || slot_mapping == nullptr || nkv == 0) return;
  __syncthreads();
  const long long slot = slot_mapping[t];
  if (slot < 0) return;                      // a padding token: stored nowhere
  if (slot >= num_pages * page_size) {
    if (threadIdx.x == 0) fmx_set_status(status, FMX_BAD_SLOT, slot, t);
    return;
  }
  const long long page = slot / page_size;
  const int off = (int)(slot - page * page_size);
  const T* ksrc = row + (long long)nh * hd;
  const T* vsrc = ksrc + (long long)nkv * hd;
  const int n = nkv * hd;
  for (int it = threadIdx.x; it < n; it += blockDim.x) {
    const int g = it / hd, e = it - g * hd;
    const long long kdst = (((page * 2 + 0) * nkv + g) * page_size + off) * hd + e;
    const long long vdst = (((page * 2 + 1) * nkv + g) * page_size + off) * hd + e;
    kv[kdst] = ksrc[it];
    kv[vdst] = vsrc[it];
  }
}

FMX_EXPORT int fmx_rope_kv_write(void* qkv, const int* positions, const float* inv_freq, const long long* slot_mapping,
                                 void* kv, int T, int nh, int nkv, int hd, int rot, int interleaved, int page_size,
                                 long long num_pages, long long row_stride, int dtype, int* status,
                                 cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || nh < 0 || nkv < 0 || hd <= 0 || rot < 0 || rot > hd || (rot & 1))
    return fmx_fail("fmx_rope_kv_write: bad sizes T=%d nh=%d nkv=%d hd=%d rot=%d", T, nh, nkv, hd, rot);
  if (rot > 0 && inv_freq == nullptr) return fmx_fail("fmx_rope_kv_write: rot=%d needs a frequency table", rot);
  if (row_stride < (long long)(nh + 2 * nkv) * hd) return fmx_fail("fmx_rope_kv_write: row stride too small");
  const int block = 128;
  if (dtype == FMX_F32)
    rope_kv_write_kernel<float><<<T, block, 0, stream>>>((float*)qkv, positions, inv_freq, slot_mapping, (float*)kv, nh,
                                                        nkv, hd, rot, interleaved, page_size, num_pages, row_stride,
                                                        status);
  else if (dtype == FMX_BF16)
    rope_kv_write_kernel<bf16><<<T, block, 0, stream>>>((bf16*)qkv, positions, inv_freq, slot_mapping, (bf16*)kv, nh,
                                                       nkv, hd, rot, interleaved, page_size, num_pages, row_stride,
                                                       status);
  else
    return fmx_fail("fmx_rope_kv_write: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}
