// Rotary position encoding fused with the write of keys and values into the paged
// cache, plus the two halves alone (rotation in place; plain cache write) for mixers
// whose position encoding is not rotary.
//
// Rotation: include/photon/ops/kernels/rope_kernel.hpp:143-165, (x0, x1) ->
// (x0*cos - x1*sin, x0*sin + x1*cos); the angle pos * inv_freq[j] and its sine and
// cosine are computed in 32-bit (same file, :76-82).  interleaved != 0 pairs
// (x[2j], x[2j+1]) as the reference does, else (x[j], x[j + d/2]).
// Cache write: src/ops/kernels/cuda/paged_kv_write.cu:26-77, with the page layout
// [page][kv_head][slot in page][head_dim] and the token's place given as
// slot = page * page_size + offset.
#include "common.cuh"

// q [T, n_q * d], k and v [T, n_kv * d], each with its own row stride in elements (they are
// usually three sections of one fused row).  q and k may be null (nothing to rotate),
// v may be null when nothing is stored.  grid: T, block: 128.  dynamic smem: d floats (cos | sin).
template <typename T>
__global__ void rope_kv_write_kernel(T* q, long q_stride, T* k, long k_stride, const T* v, long v_stride,
                                     const int* __restrict__ positions,
                                     const float* __restrict__ inv_freq, int interleaved,
                                     const int* __restrict__ slot_mapping, T* __restrict__ k_cache,
                                     T* __restrict__ v_cache, int n_q, int n_kv, int d, int page_size,
                                     long num_slots, int rotate, int write_kv, int* err) {
  extern __shared__ float cs[];
  const int t = blockIdx.x;
  const int half = d >> 1;
  float* cosv = cs;
  float* sinv = cs + half;
  if (rotate) {
    const float pos = (float)positions[t];
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      float s, c;
      sincosf(pos * inv_freq[j], &s, &c);
      cosv[j] = c;
      sinv[j] = s;
    }
    __syncthreads();
  }
  T* row = q ? q + (size_t)t * q_stride : nullptr;
  // queries: rotate in place
  if (rotate && row) {
    const int pairs = n_q * half;
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
      const int h = p / half, j = p - h * half;
      const int i0 = interleaved ? h * d + 2 * j : h * d + j;
      const int i1 = interleaved ? i0 + 1 : i0 + half;
      const float x0 = to_f32(row[i0]), x1 = to_f32(row[i1]);
      row[i0] = from_f32<T>(x0 * cosv[j] - x1 * sinv[j]);
      row[i1] = from_f32<T>(x0 * sinv[j] + x1 * cosv[j]);
    }
  }
  // keys: rotate, then store in the row (so that a caller that does not use the cache sees
  // them) and in the cache; values: copy
  long slot = -1;
  if (write_kv) {
    slot = slot_mapping[t];
    if (slot >= num_slots || slot < -1) {
      if (threadIdx.x == 0) report_error(err, PHOTON_DEV_BAD_SLOT, t, (int)slot, (int)num_slots);
      slot = -1;
    }
  }
  const long page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? (int)(slot - page * page_size) : 0;
  if (k == nullptr) return;
  T* krow = k + (size_t)t * k_stride;
  const T* vrow = v ? v + (size_t)t * v_stride : nullptr;
  if (vrow == nullptr) slot = -1;
  const int kpairs = n_kv * half;
  for (int p = threadIdx.x; p < kpairs; p += blockDim.x) {
    const int h = p / half, j = p - h * half;
    const int i0 = interleaved ? 2 * j : j;
    const int i1 = interleaved ? i0 + 1 : i0 + half;
    float x0 = to_f32(krow[h * d + i0]), x1 = to_f32(krow[h * d + i1]);
    T y0, y1;
    if (rotate) {
      y0 = from_f32<T>(x0 * cosv[j] - x1 * sinv[j]);
      y1 = from_f32<T>(x0 * sinv[j] + x1 * cosv[j]);
      krow[h * d + i0] = y0;
      krow[h * d + i1] = y1;
    } else {
      y0 = krow[h * d + i0];
      y1 = krow[h * d + i1];
    }
    if (slot >= 0) {
      const size_t base = (((size_t)page * n_kv + h) * page_size + off) * d;
      k_cache[base + i0] = y0;
      k_cache[base + i1] = y1;
      v_cache[base + i0] = vrow[h * d + i0];
      v_cache[base + i1] = vrow[h * d + i1];
    }
  }
}

// rotate: apply the rotation to q and k.  write_kv: store k and v at slot_mapping.
PHOTON_API int photon_rope_kv_write(void* q, long q_stride, void* k, long k_stride, const void* v,
                                    long v_stride, int dtype, const int* positions,
                                    const float* inv_freq, int interleaved, const int* slot_mapping,
                                    void* k_cache, void* v_cache, int T, int n_q, int n_kv, int d,
                                    int page_size, long num_slots, int rotate, int write_kv, int* err,
                                    cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d <= 0 || (d & 1)) return PHOTON_ERR_UNSUPPORTED;
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 48 * 1024) return PHOTON_ERR_UNSUPPORTED;
  if (dtype == PHOTON_BF16)
    rope_kv_write_kernel<bf16><<<T, 128, smem, stream>>>((bf16*)q, q_stride, (bf16*)k, k_stride,
        (const bf16*)v, v_stride, positions, inv_freq,
        interleaved, slot_mapping, (bf16*)k_cache, (bf16*)v_cache, n_q, n_kv, d, page_size, num_slots,
        rotate, write_kv, err);
  else
    rope_kv_write_kernel<float><<<T, 128, smem, stream>>>((float*)q, q_stride, (float*)k, k_stride,
        (const float*)v, v_stride, positions, inv_freq,
        interleaved, slot_mapping, (float*)k_cache, (float*)v_cache, n_q, n_kv, d, page_size, num_slots,
        rotate, write_kv, err);
  return launch_status();
}
