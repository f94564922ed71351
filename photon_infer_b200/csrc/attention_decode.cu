// Paged attention for tokens that read a long cache and bring little work of their own
// (decoded tokens, short prompt portions): the keys of one token are split over several
// blocks, each block streams its share of keys and values once with 16-byte loads and
// keeps a running softmax in 32-bit, a second kernel merges the shares.
//
// Compiled per model: -DHEAD_DIM=<d> -DGROUP=<query heads per key/value head>.
// Formula as in attention.cu (include/photon/ops/kernels/mha_kernel.hpp:188-229): scores
// (q.k)/sqrt(d) over the keys max(0, p-window+1)..p, softmax exp(s-max)/sum, sum of p*v.
//
// Layout of work: a key row of HEAD_DIM elements is read by LPK = HEAD_DIM/VEC lanes
// (VEC = 16 bytes of elements), so a warp reads 32/LPK keys at once, fully coalesced.
// Every lane group keeps its own running (max, sum, accumulator) for the GROUP heads;
// groups are merged through shared memory at the end.
//
// Scratch: the shares are written to `part_acc` [T, n_q, splits, HEAD_DIM] and
// `part_ml` [T, n_q, splits, 2] (float), both given by the caller.
#include "common.cuh"
#include <math.h>

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
#ifndef GROUP
#define GROUP 4
#endif

#define DEC_WARPS 4
#define DEC_THREADS (DEC_WARPS * 32)
#if GROUP > 4
#define DEC_KC 2                      // keys per lane group per round
#else
#define DEC_KC 4
#endif
// float storage reads 4 elements per lane: head sizes above 128 would need more than a warp per key
#if HEAD_DIM <= 128
#define DEC_HAS_F32 1
#else
#define DEC_HAS_F32 0
#endif

template <typename T> struct Vec16;
template <> struct Vec16<bf16> {
  static constexpr int N = 8;
  __device__ static float exp_(float x) { return __expf(x); }
  __device__ static void load(const bf16* p, float* f) {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 x = __bfloat1622float2(h[i]); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
  }
};
template <> struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static float exp_(float x) { return expf(x); }
  __device__ static void load(const float* p, float* f) {
    const float4 r = __ldg(reinterpret_cast<const float4*>(p));
    f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w;
  }
};

template <typename T>
__global__ void __launch_bounds__(DEC_THREADS)
decode_attention_kernel(const T* __restrict__ q, long q_stride, T* __restrict__ out, long out_stride,
                        const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                        const int* __restrict__ block_table, int max_pages, const int* __restrict__ token_seq,
                        const int* __restrict__ positions, float* __restrict__ part_acc,
                        float* __restrict__ part_ml, int n_kv, int page_size, int num_pages, int window,
                        float scale, int num_splits, int* err) {
  constexpr int VEC = Vec16<T>::N;
  constexpr int LPK = HEAD_DIM / VEC;             // lanes per key row
  constexpr int KPW = 32 / LPK;                   // keys per warp and load
  constexpr int NG = DEC_WARPS * KPW;             // lane groups per block
  constexpr int ROUND = NG * DEC_KC;              // keys per block and round
  static_assert(HEAD_DIM % VEC == 0 && (LPK & (LPK - 1)) == 0 && LPK <= 32 && LPK >= 1, "head size");

  __shared__ float s_m[NG][GROUP];
  __shared__ float s_l[NG][GROUP];
  __shared__ float s_acc[NG][GROUP][HEAD_DIM];

  const int split = blockIdx.x, g = blockIdx.y, t = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / LPK, li = lane % LPK;
  const int grp = warp * KPW + sub;
  const int n_q = n_kv * GROUP;

  const int p = positions[t];
  const int seq = token_seq[t];
  const int kstart = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int kend = p + 1;
  int per = (kend - kstart + num_splits - 1) / num_splits;
  per = (per + ROUND - 1) / ROUND * ROUND;
  const int begin = kstart + split * per;
  const int end = min(kend, begin + per);
  const int* table = block_table + (size_t)seq * max_pages;

  float qf[GROUP][VEC];
#pragma unroll
  for (int h = 0; h < GROUP; ++h)
    Vec16<T>::load(q + (size_t)t * q_stride + (size_t)(g * GROUP + h) * HEAD_DIM + li * VEC, qf[h]);

  float m[GROUP], l[GROUP], acc[GROUP][VEC];
#pragma unroll
  for (int h = 0; h < GROUP; ++h) {
    m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[h][i] = 0.f;
  }

  for (int base = begin; base < end; base += ROUND) {
    long long off[DEC_KC];
    float kf[DEC_KC][VEC];
#pragma unroll
    for (int c = 0; c < DEC_KC; ++c) {
      const int key = base + c * NG + grp;
      off[c] = -1;
      if (key < end) {
        const int page = table[key / page_size];
        if (page < 0 || page >= num_pages) {
          if (li == 0) report_error(err, PHOTON_DEV_BAD_PAGE, t, key, page);
        } else {
          off[c] = (((long long)page * n_kv + g) * page_size + (key % page_size)) * HEAD_DIM + li * VEC;
        }
      }
      if (off[c] >= 0) Vec16<T>::load(k_cache + off[c], kf[c]);
    }
    float s[DEC_KC][GROUP];
#pragma unroll
    for (int c = 0; c < DEC_KC; ++c)
#pragma unroll
      for (int h = 0; h < GROUP; ++h) {
        float d = 0.f;
        if (off[c] >= 0) {
#pragma unroll
          for (int i = 0; i < VEC; ++i) d += qf[h][i] * kf[c][i];
        }
#pragma unroll
        for (int o = LPK >> 1; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        s[c][h] = off[c] >= 0 ? d * scale : -INFINITY;
      }
    // values of the same keys (loads are issued before the exponentials are needed)
    float vf[DEC_KC][VEC];
#pragma unroll
    for (int c = 0; c < DEC_KC; ++c) {
      if (off[c] >= 0) {
        Vec16<T>::load(v_cache + off[c], vf[c]);
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) vf[c][i] = 0.f;
      }
    }
#pragma unroll
    for (int h = 0; h < GROUP; ++h) {
      float mx = s[0][h];
#pragma unroll
      for (int c = 1; c < DEC_KC; ++c) mx = fmaxf(mx, s[c][h]);
      const float m_new = fmaxf(m[h], mx);
      if (m_new == -INFINITY) continue;                    // no key of this group yet
      const float corr = (m[h] == -INFINITY) ? 0.f : Vec16<T>::exp_(m[h] - m_new);
      m[h] = m_new;
      l[h] *= corr;
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[h][i] *= corr;
#pragma unroll
      for (int c = 0; c < DEC_KC; ++c) {
        const float pr = (s[c][h] == -INFINITY) ? 0.f : Vec16<T>::exp_(s[c][h] - m_new);
        l[h] += pr;
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[h][i] += pr * vf[c][i];
      }
    }
  }

  // merge the lane groups of the block
  if (li == 0) {
#pragma unroll
    for (int h = 0; h < GROUP; ++h) { s_m[grp][h] = m[h]; s_l[grp][h] = l[h]; }
  }
#pragma unroll
  for (int h = 0; h < GROUP; ++h)
#pragma unroll
    for (int i = 0; i < VEC; ++i) s_acc[grp][h][li * VEC + i] = acc[h][i];
  __syncthreads();
  for (int e = threadIdx.x; e < GROUP * HEAD_DIM; e += DEC_THREADS) {
    const int h = e / HEAD_DIM, d = e - h * HEAD_DIM;
    float M = -INFINITY;
#pragma unroll
    for (int x = 0; x < NG; ++x) M = fmaxf(M, s_m[x][h]);
    float L = 0.f, A = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int x = 0; x < NG; ++x) {
        const float w = (s_m[x][h] == -INFINITY) ? 0.f : Vec16<T>::exp_(s_m[x][h] - M);
        L += s_l[x][h] * w;
        A += s_acc[x][h][d] * w;
      }
    }
    const int head = g * GROUP + h;
    if (num_splits == 1) {
      out[(size_t)t * out_stride + (size_t)head * HEAD_DIM + d] = from_f32<T>(L > 0.f ? A / L : 0.f);
    } else {
      const size_t slot = ((size_t)t * n_q + head) * num_splits + split;
      part_acc[slot * HEAD_DIM + d] = A;
      if (d == 0) { part_ml[slot * 2] = M; part_ml[slot * 2 + 1] = L; }
    }
  }
}

// grid (T, n_q), HEAD_DIM threads (at least 32)
template <typename T>
__global__ void decode_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                    T* __restrict__ out, long out_stride, int n_q, int num_splits) {
  const int t = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
  if (d >= HEAD_DIM) return;
  const size_t base = ((size_t)t * n_q + head) * num_splits;
  float M = -INFINITY;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
  float L = 0.f, A = 0.f;
  if (M != -INFINITY) {
    for (int s = 0; s < num_splits; ++s) {
      const float ms = part_ml[(base + s) * 2];
      const float w = (ms == -INFINITY) ? 0.f : expf(ms - M);
      L += part_ml[(base + s) * 2 + 1] * w;
      A += part_acc[(base + s) * HEAD_DIM + d] * w;
    }
  }
  out[(size_t)t * out_stride + (size_t)head * HEAD_DIM + d] = from_f32<T>(L > 0.f ? A / L : 0.f);
}

template <typename T>
static int decode_launch(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                         const void* v_cache, const int* block_table, int max_pages, const int* token_seq,
                         const int* positions, float* part_acc, float* part_ml, int T_, int n_kv, int page_size,
                         int num_pages, int window, float scale, int num_splits, int* err, cudaStream_t stream) {
  dim3 grid(num_splits, n_kv, T_);
  decode_attention_kernel<T><<<grid, DEC_THREADS, 0, stream>>>(
      (const T*)q, q_stride, (T*)out, out_stride, (const T*)k_cache, (const T*)v_cache, block_table, max_pages,
      token_seq, positions, part_acc, part_ml, n_kv, page_size, num_pages, window, scale, num_splits, err);
  int st = launch_status();
  if (st != 0 || num_splits == 1) return st;
  dim3 mgrid(T_, n_kv * GROUP);
  decode_merge_kernel<T><<<mgrid, HEAD_DIM < 32 ? 32 : HEAD_DIM, 0, stream>>>(part_acc, part_ml, (T*)out,
                                                                              out_stride, n_kv * GROUP, num_splits);
  return launch_status();
}

PHOTON_API int photon_decode_attention_head_dim() { return HEAD_DIM; }
PHOTON_API int photon_decode_attention_group() { return GROUP; }

// part_acc: float [T * n_q * num_splits * HEAD_DIM]; part_ml: float [T * n_q * num_splits * 2]; both may be
// null when num_splits == 1.  q rows must be 16-byte aligned (q_stride * sizeof(T) a multiple of 16).
PHOTON_API int photon_decode_attention(const void* q, long q_stride, void* out, long out_stride, int dtype,
                                       const void* k_cache, const void* v_cache, const int* block_table,
                                       int max_pages, const int* token_seq, const int* positions,
                                       float* part_acc, float* part_ml, int T_, int n_q, int n_kv, int d,
                                       int page_size, int num_pages, int window, float scale, int num_splits,
                                       int* err, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (d != HEAD_DIM || n_kv <= 0 || n_q != n_kv * GROUP) return PHOTON_ERR_UNSUPPORTED;
  if (num_splits < 1 || num_splits > 65535 || n_kv > 65535 || T_ > 65535) return PHOTON_ERR_UNSUPPORTED;
  if (num_splits > 1 && (part_acc == nullptr || part_ml == nullptr)) return PHOTON_ERR_ARGUMENT;
  const size_t esz = dtype == PHOTON_BF16 ? 2 : 4;
  if (((size_t)q_stride * esz) % 16 || ((uintptr_t)q % 16) || ((uintptr_t)k_cache % 16) || ((uintptr_t)v_cache % 16))
    return PHOTON_ERR_ARGUMENT;
  if (dtype == PHOTON_BF16)
    return decode_launch<bf16>(q, q_stride, out, out_stride, k_cache, v_cache, block_table, max_pages, token_seq,
                               positions, part_acc, part_ml, T_, n_kv, page_size, num_pages, window, scale,
                               num_splits, err, stream);
#if DEC_HAS_F32
  return decode_launch<float>(q, q_stride, out, out_stride, k_cache, v_cache, block_table, max_pages, token_seq,
                              positions, part_acc, part_ml, T_, n_kv, page_size, num_pages, window, scale,
                              num_splits, err, stream);
#else
  return PHOTON_ERR_UNSUPPORTED;
#endif
}
