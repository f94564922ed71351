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
// v may be null when nothing is stored.
// One thread per pair of elements: items [0, n_q*d/2) rotate a pair of q in place, the next
// n_kv*d/2 rotate a pair of k (in place and into the cache), the last n_kv*d/2 copy a pair of v
// into the cache.  grid: (ceil(items / 128), T), block: 128.  No shared memory, no barrier; a
// thread computes the sine and cosine of its own angle.
template <typename T>
__global__ void __launch_bounds__(128)
rope_kv_write_kernel(T* q, long q_stride, T* k, long k_stride, const T* v, long v_stride,
                     const int* __restrict__ positions, const float* __restrict__ inv_freq, int interleaved,
                     const int* __restrict__ slot_mapping, T* __restrict__ k_cache, T* __restrict__ v_cache,
                     int n_q, int n_kv, int d, int page_size, long num_slots, int rotate, int write_kv,
                     int* err) {
  const int t = blockIdx.y;
  const int half = d >> 1;
  const int item = blockIdx.x * blockDim.x + threadIdx.x;
  const int q_items = q ? n_q * half : 0;
  const int k_items = k ? n_kv * half : 0;
  const int v_items = (v && write_kv) ? n_kv * half : 0;
  if (item >= q_items + k_items + v_items) return;

  int which, local;                       // 0 q, 1 k, 2 v
  if (item < q_items) { which = 0; local = item; }
  else if (item < q_items + k_items) { which = 1; local = item - q_items; }
  else { which = 2; local = item - q_items - k_items; }
  const int h = local / half, j = local - h * half;
  const int i0 = (which != 2 && !interleaved) ? j : 2 * j;
  const int i1 = (which != 2 && !interleaved) ? j + half : 2 * j + 1;

  long slot = -1;
  if (which != 0 && write_kv) {
    slot = slot_mapping[t];
    if (slot >= num_slots || slot < -1) {
      if (local == 0 && which == 1) report_error(err, PHOTON_DEV_BAD_SLOT, t, (int)slot, (int)num_slots);
      slot = -1;
    }
  }
  size_t cache_at = 0;
  if (slot >= 0) {
    const long page = slot / page_size;
    const int off = (int)(slot - page * page_size);
    cache_at = (((size_t)page * n_kv + h) * page_size + off) * d;
  }
  if (which == 2) {
    if (slot >= 0) {
      const T* vrow = v + (size_t)t * v_stride + (size_t)h * d;
      v_cache[cache_at + i0] = vrow[i0];
      v_cache[cache_at + i1] = vrow[i1];
    }
    return;
  }
  T* row = (which == 0 ? q + (size_t)t * q_stride : k + (size_t)t * k_stride) + (size_t)h * d;
  T y0 = row[i0], y1 = row[i1];
  if (rotate) {
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[j], &sn, &cs);
    const float x0 = to_f32(y0), x1 = to_f32(y1);
    y0 = from_f32<T>(x0 * cs - x1 * sn);
    y1 = from_f32<T>(x0 * sn + x1 * cs);
    row[i0] = y0;
    row[i1] = y1;
  }
  if (which == 1 && slot >= 0) {
    k_cache[cache_at + i0] = y0;
    k_cache[cache_at + i1] = y1;
  }
}

// The same work for bfloat16 rows whose head size is a multiple of 16, 16 bytes per access: an item
// is 8 pairs (two 16-byte pieces of one head).  Needs 16-byte aligned rows and caches.
__global__ void __launch_bounds__(128)
rope_kv_write_vec_kernel(bf16* q, long q_stride, bf16* k, long k_stride, const bf16* v, long v_stride,
                         const int* __restrict__ positions, const float* __restrict__ inv_freq, int interleaved,
                         const int* __restrict__ slot_mapping, bf16* __restrict__ k_cache,
                         bf16* __restrict__ v_cache, int n_q, int n_kv, int d, int page_size, long num_slots,
                         int rotate, int write_kv, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.y;
  const int per_head = d >> 4;                               // items per head
  const int item = blockIdx.x * blockDim.x + threadIdx.x;
  const int q_items = q ? n_q * per_head : 0;
  const int k_items = k ? n_kv * per_head : 0;
  const int v_items = (v && write_kv) ? n_kv * per_head : 0;
  if (item >= q_items + k_items + v_items) return;
  int which, local;
  if (item < q_items) { which = 0; local = item; }
  else if (item < q_items + k_items) { which = 1; local = item - q_items; }
  else { which = 2; local = item - q_items - k_items; }
  const int h = local / per_head, a = local - h * per_head;
  const int half = d >> 1;
  // element offsets of the two 16-byte pieces inside the head, and the first pair index
  const int e0 = (which == 2 || interleaved) ? a * 16 : a * 8;
  const int e1 = (which == 2 || interleaved) ? a * 16 + 8 : half + a * 8;
  const int j0 = a * 8;

  long slot = -1;
  if (which != 0 && write_kv) {
    slot = slot_mapping[t];
    if (slot >= num_slots || slot < -1) {
      if (local == 0 && which == 1) report_error(err, PHOTON_DEV_BAD_SLOT, t, (int)slot, (int)num_slots);
      slot = -1;
    }
  }
  size_t cache_at = 0;
  if (slot >= 0) {
    const long page = slot / page_size;
    const int off = (int)(slot - page * page_size);
    cache_at = (((size_t)page * n_kv + h) * page_size + off) * d;
  }
  if (which == 2) {
    if (slot >= 0) {
      const bf16* vrow = v + (size_t)t * v_stride + (size_t)h * d;
      *reinterpret_cast<uint4*>(v_cache + cache_at + e0) = *reinterpret_cast<const uint4*>(vrow + e0);
      *reinterpret_cast<uint4*>(v_cache + cache_at + e1) = *reinterpret_cast<const uint4*>(vrow + e1);
    }
    return;
  }
  bf16* row = (which == 0 ? q + (size_t)t * q_stride : k + (size_t)t * k_stride) + (size_t)h * d;
  uint4 r0 = *reinterpret_cast<const uint4*>(row + e0);
  uint4 r1 = *reinterpret_cast<const uint4*>(row + e1);
  if (rotate) {
    bf16* p0 = reinterpret_cast<bf16*>(&r0);
    bf16* p1 = reinterpret_cast<bf16*>(&r1);
    const float pos = (float)positions[t];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float sn, cs;
      sincosf(pos * inv_freq[j0 + e], &sn, &cs);
      // pair e of the item: (p0[e], p1[e]) when halves are paired, neighbours of the 16 elements otherwise
      bf16* x0 = interleaved ? (e < 4 ? p0 + 2 * e : p1 + 2 * (e - 4)) : p0 + e;
      bf16* x1 = interleaved ? x0 + 1 : p1 + e;
      const float a0 = __bfloat162float(*x0), a1 = __bfloat162float(*x1);
      *x0 = __float2bfloat16_rn(a0 * cs - a1 * sn);
      *x1 = __float2bfloat16_rn(a0 * sn + a1 * cs);
    }
    *reinterpret_cast<uint4*>(row + e0) = r0;
    *reinterpret_cast<uint4*>(row + e1) = r1;
  }
  if (which == 1 && slot >= 0) {
    *reinterpret_cast<uint4*>(k_cache + cache_at + e0) = r0;
    *reinterpret_cast<uint4*>(k_cache + cache_at + e1) = r1;
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
  const int items = ((q ? n_q : 0) + (k ? n_kv : 0) + ((v && write_kv) ? n_kv : 0)) * (d / 2);
  if (items <= 0) return 0;
  if (T > 65535) return PHOTON_ERR_UNSUPPORTED;
  dim3 grid((items + 127) / 128, T);
  const bool aligned = ((uintptr_t)q % 16 == 0) && ((uintptr_t)k % 16 == 0) && ((uintptr_t)v % 16 == 0) &&
                       ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0) && (q_stride % 8 == 0) &&
                       (k_stride % 8 == 0) && (v_stride % 8 == 0);
  if (dtype == PHOTON_BF16 && d % 16 == 0 && aligned) {
    const int vitems = ((q ? n_q : 0) + (k ? n_kv : 0) + ((v && write_kv) ? n_kv : 0)) * (d / 16);
    dim3 vgrid((vitems + 127) / 128, T);
    return launch_pdl(rope_kv_write_vec_kernel, vgrid, dim3(128), 0, stream, (bf16*)q, q_stride, (bf16*)k, k_stride,
                      (const bf16*)v, v_stride, positions, inv_freq, interleaved, slot_mapping, (bf16*)k_cache,
                      (bf16*)v_cache, n_q, n_kv, d, page_size, num_slots, rotate, write_kv, err);
  }
  if (dtype == PHOTON_BF16)
    rope_kv_write_kernel<bf16><<<grid, 128, 0, stream>>>((bf16*)q, q_stride, (bf16*)k, k_stride,
        (const bf16*)v, v_stride, positions, inv_freq,
        interleaved, slot_mapping, (bf16*)k_cache, (bf16*)v_cache, n_q, n_kv, d, page_size, num_slots,
        rotate, write_kv, err);
  else
    rope_kv_write_kernel<float><<<grid, 128, 0, stream>>>((float*)q, q_stride, (float*)k, k_stride,
        (const float*)v, v_stride, positions, inv_freq,
        interleaved, slot_mapping, (float*)k_cache, (float*)v_cache, n_q, n_kv, d, page_size, num_slots,
        rotate, write_kv, err);
  return launch_status();
}

// Table of (cos, sin) of position * inv_freq[j] for positions 0 .. count - 1: the same expression, in the same
// 32-bit arithmetic, that the kernels above evaluate in place, so a kernel that reads the table rotates
// exactly as they do.  out: float2 [count, half].
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, int half, long total, float2* __restrict__ out) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long p = i / half;
  const int j = (int)(i - p * half);
  float sn, cs;
  sincosf((float)p * inv_freq[j], &sn, &cs);
  out[i] = make_float2(cs, sn);
}

PHOTON_API int photon_rope_table(const float* inv_freq, int half, int count, void* out, cudaStream_t stream) {
  if (half <= 0 || count <= 0) return 0;
  const long total = (long)half * count;
  rope_table_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(inv_freq, half, total, (float2*)out);
  return launch_status();
}
