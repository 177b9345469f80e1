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
      float x, y;
      rope_pair(a, b, s, c, x, y);
      p[i0] = from_f<T>(x);
      p[i1] = from_f<T>(y);
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

// bfloat16, half-split pairing, rot/2 and hd multiples of 8, 16-byte aligned rows: sine and
// cosine once per (token, pair) in shared memory, eight pairs per thread with 16-byte
// accesses, and the rotated k (and v) written to the page in the same pass.
__global__ void __launch_bounds__(128)
rope_kv_write_bf16_vec_kernel(bf16* qkv, const int* positions, const float* __restrict__ inv_freq,
                              const long long* slot_mapping, bf16* kv, int nh, int nkv, int hd, int rot,
                              int page_size, long long num_pages, long long row_stride, int* status) {
  extern __shared__ float sc[];                 // [half] sines, [half] cosines
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  bf16* row = qkv + (long long)t * row_stride;
  const int half = rot / 2;
  const float pos = (float)positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &sc[j], &sc[half + j]);
  long long slot = (kv != nullptr && slot_mapping != nullptr && nkv > 0) ? slot_mapping[t] : -1;
  if (slot >= num_pages * page_size) {
    if (threadIdx.x == 0) fmx_set_status(status, FMX_BAD_SLOT, slot, t);
    slot = -1;
  }
  const long long page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? (int)(slot - page * page_size) : 0;
  __syncthreads();
  const int hv = half / 8;                      // vector items per head for the rotated part
  const int pv = (hd - rot) / 8;                // and for the part that is not rotated
  const int per_head = hv + pv;
  const int items = (nh + nkv) * per_head + nkv * (hd / 8);
  for (int it = threadIdx.x; it < items; it += blockDim.x) {
    if (it < (nh + nkv) * per_head) {
      const int h = it / per_head, c = it - h * per_head;
      bf16* p = row + (long long)h * hd;
      bf16* dst = nullptr;
      if (h >= nh && slot >= 0) dst = kv + ((((page * 2 + 0) * nkv + (h - nh)) * page_size + off) * (long long)hd);
      if (c < hv) {
        uint4 a = *reinterpret_cast<uint4*>(p + 8 * c), b = *reinterpret_cast<uint4*>(p + half + 8 * c);
        __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&a);
        __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 fa = __bfloat1622float2(a2[e]), fb = __bfloat1622float2(b2[e]);
          const int j = 8 * c + 2 * e;
          const float s0 = sc[j], c0 = sc[half + j], s1 = sc[j + 1], c1 = sc[half + j + 1];
          float x0, y0, x1, y1;
          rope_pair(fa.x, fb.x, s0, c0, x0, y0);
          rope_pair(fa.y, fb.y, s1, c1, x1, y1);
          a2[e] = __floats2bfloat162_rn(x0, x1);
          b2[e] = __floats2bfloat162_rn(y0, y1);
        }
        *reinterpret_cast<uint4*>(p + 8 * c) = a;
        *reinterpret_cast<uint4*>(p + half + 8 * c) = b;
        if (dst) {
          *reinterpret_cast<uint4*>(dst + 8 * c) = a;
          *reinterpret_cast<uint4*>(dst + half + 8 * c) = b;
        }
      } else if (dst) {
        const int e0 = rot + 8 * (c - hv);
        *reinterpret_cast<uint4*>(dst + e0) = *reinterpret_cast<const uint4*>(p + e0);
      }
    } else if (slot >= 0) {
      const int iv = it - (nh + nkv) * per_head;
      const int g = iv / (hd / 8), c = iv - g * (hd / 8);
      const bf16* src = row + (long long)(nh + nkv + g) * hd + 8 * c;
      bf16* dst = kv + ((((page * 2 + 1) * nkv + g) * page_size + off) * (long long)hd) + 8 * c;
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
    }
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
  else if (dtype == FMX_BF16) {
    const bool vec = !interleaved && rot > 0 && rot % 16 == 0 && hd % 8 == 0 && row_stride % 8 == 0 &&
                     ((uintptr_t)qkv & 15) == 0 && (kv == nullptr || ((uintptr_t)kv & 15) == 0);
    if (vec)
      fmx_launch(rope_kv_write_bf16_vec_kernel, dim3(T), dim3(block), (size_t)rot * sizeof(float), stream,
          (bf16*)qkv, positions, inv_freq, slot_mapping, (bf16*)kv, nh, nkv, hd, rot, page_size, num_pages, row_stride,
          status);
    else
      rope_kv_write_kernel<bf16><<<T, block, 0, stream>>>((bf16*)qkv, positions, inv_freq, slot_mapping, (bf16*)kv, nh,
                                                         nkv, hd, rot, interleaved, page_size, num_pages, row_stride,
                                                         status);
  }
  else
    return fmx_fail("fmx_rope_kv_write: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}
