// Paged causal attention with grouped heads, the general kernel: any head size that
// is even, any number of heads and groups, any page size, float or bfloat16 storage,
// an optional window.  One block handles one token of the step and one key/value head
// (all query heads of that group), walks the keys in tiles of 32 from the cache and
// keeps a running softmax in 32-bit.  Prompt portions and single decoded tokens are
// the same case: a token at position p of its request sees the keys
// max(0, p - window + 1) .. p, which the cache holds once this step's keys are written.
//
// Formula: include/photon/ops/kernels/mha_kernel.hpp:188-229 (scores (q.k)/sqrt(d) for
// keys <= pos only, softmax exp(s - max)/sum, weighted sum of values; query head h
// uses key/value head h / (n_q / n_kv)).  The reference's paged kernel
// (src/ops/kernels/cuda/paged_attention.cu:90-194) adds 1e-6 to the denominator and
// lets a token see later tokens of its own portion; neither is done here.
//
// The tile grid starts at key 0 (at a multiple of 32 at or below the window's first
// key), so the order of every sum depends only on the token's position, never on how
// the request was cut into steps or on what else is in the batch.
#include "common.cuh"
#include <math.h>

#define ATT_TILE 32
#define ATT_THREADS 128

template <typename T, int PPT>
__global__ void __launch_bounds__(ATT_THREADS)
paged_attention_kernel(const T* __restrict__ q, long q_stride, T* __restrict__ out, long out_stride,
                       const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                       const int* __restrict__ block_table, int max_pages,
                       const int* __restrict__ token_seq, const int* __restrict__ positions,
                       int n_q, int n_kv, int d, int page_size, int num_pages, int window, float scale,
                       int* err) {
  extern __shared__ __align__(16) float smem[];
  const int t = blockIdx.x, g = blockIdx.y;
  const int G = n_q / n_kv;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* qs = smem;                          // G * d
  float* ks = qs + G * d;                    // TILE * (d + 1)
  float* vs = ks + ATT_TILE * (d + 1);       // TILE * d
  float* sc = vs + ATT_TILE * d;             // G * TILE
  float* mrun = sc + G * ATT_TILE;           // G
  float* lsum = mrun + G;                    // G
  float* corr = lsum + G;                    // G
  long long* kbase = (long long*)(corr + G + ((G & 1) ? 1 : 0));   // TILE (8-byte aligned)

  const int p = positions[t];
  const int seq = token_seq[t];
  const int kstart = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int* table = block_table + (size_t)seq * max_pages;

  for (int i = tid; i < G * d; i += ATT_THREADS) {
    const int h = i / d, j = i - h * d;
    qs[i] = to_f32(q[(size_t)t * q_stride + (size_t)(g * G + h) * d + j]);
  }
  for (int h = tid; h < G; h += ATT_THREADS) { mrun[h] = -INFINITY; lsum[h] = 0.f; corr[h] = 0.f; }
  float acc[PPT];
#pragma unroll
  for (int n = 0; n < PPT; ++n) acc[n] = 0.f;

  for (int tile0 = (kstart / ATT_TILE) * ATT_TILE; tile0 <= p; tile0 += ATT_TILE) {
    __syncthreads();                          // previous tile fully consumed; qs ready on the first pass
    if (tid < ATT_TILE) {
      const int kk = tile0 + tid;
      long long base = -1;
      if (kk >= kstart && kk <= p) {
        const int page = table[kk / page_size];
        if (page < 0 || page >= num_pages) {
          report_error(err, PHOTON_DEV_BAD_PAGE, t, kk, page);
        } else {
          base = (((long long)page * n_kv + g) * page_size + (kk % page_size)) * d;
        }
      }
      kbase[tid] = base;
    }
    __syncthreads();
    for (int i = tid; i < ATT_TILE * d; i += ATT_THREADS) {
      const int key = i / d, j = i - key * d;
      const long long base = kbase[key];
      ks[key * (d + 1) + j] = base >= 0 ? to_f32(k_cache[base + j]) : 0.f;
      vs[key * d + j] = base >= 0 ? to_f32(v_cache[base + j]) : 0.f;
    }
    __syncthreads();
    // scores
    for (int i = tid; i < G * ATT_TILE; i += ATT_THREADS) {
      const int h = i / ATT_TILE, key = i - h * ATT_TILE;
      float s = -INFINITY;
      if (kbase[key] >= 0) {
        const float* qh = qs + h * d;
        const float* kr = ks + key * (d + 1);
        float dot = 0.f;
        for (int j = 0; j < d; ++j) dot += qh[j] * kr[j];
        s = dot * scale;
      }
      sc[i] = s;
    }
    __syncthreads();
    // running softmax, one warp per head, one lane per key of the tile
    for (int h = warp; h < G; h += ATT_THREADS / 32) {
      const float s = sc[h * ATT_TILE + lane];
      const float tmax = warp_max(s);
      const float m_old = mrun[h];
      const float m_new = fmaxf(m_old, tmax);
      const float pr = (s == -INFINITY) ? 0.f : expf(s - m_new);
      const float psum = warp_sum(pr);
      const float c = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
      __syncwarp();
      sc[h * ATT_TILE + lane] = pr;
      if (lane == 0) { mrun[h] = m_new; lsum[h] = lsum[h] * c + psum; corr[h] = c; }
    }
    __syncthreads();
    // weighted values
#pragma unroll
    for (int n = 0; n < PPT; ++n) {
      const int i = tid + n * ATT_THREADS;
      if (i < G * d) {
        const int h = i / d, j = i - h * d;
        float a = acc[n] * corr[h];
        const float* pr = sc + h * ATT_TILE;
#pragma unroll 8
        for (int key = 0; key < ATT_TILE; ++key) a += pr[key] * vs[key * d + j];
        acc[n] = a;
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int n = 0; n < PPT; ++n) {
    const int i = tid + n * ATT_THREADS;
    if (i < G * d) {
      const int h = i / d, j = i - h * d;
      const float l = lsum[h];
      out[(size_t)t * out_stride + (size_t)(g * G + h) * d + j] = from_f32<T>(l > 0.f ? acc[n] / l : 0.f);
    }
  }
}

template <typename T, int PPT>
static int attention_launch(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                            const void* v_cache, const int* block_table, int max_pages, const int* token_seq,
                            const int* positions, int T_, int n_q, int n_kv, int d, int page_size,
                            int num_pages, int window, float scale, int* err, cudaStream_t stream) {
  const int G = n_q / n_kv;
  const size_t floats = (size_t)G * d + ATT_TILE * (d + 1) + ATT_TILE * d + (size_t)G * ATT_TILE + 3 * G + 1;
  const size_t smem = floats * sizeof(float) + ATT_TILE * sizeof(long long) + 8;
  if (smem > 220 * 1024) return PHOTON_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(paged_attention_kernel<T, PPT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(T_, n_kv);
  paged_attention_kernel<T, PPT><<<grid, ATT_THREADS, smem, stream>>>(
      (const T*)q, q_stride, (T*)out, out_stride, (const T*)k_cache, (const T*)v_cache, block_table,
      max_pages, token_seq, positions, n_q, n_kv, d, page_size, num_pages, window, scale, err);
  return launch_status();
}

#define ATT_DISPATCH(TYPE)                                                                              \
  if (ppt <= 1) return attention_launch<TYPE, 1>(ATT_ARGS);                                             \
  if (ppt <= 2) return attention_launch<TYPE, 2>(ATT_ARGS);                                             \
  if (ppt <= 4) return attention_launch<TYPE, 4>(ATT_ARGS);                                             \
  if (ppt <= 8) return attention_launch<TYPE, 8>(ATT_ARGS);                                             \
  if (ppt <= 16) return attention_launch<TYPE, 16>(ATT_ARGS);                                           \
  if (ppt <= 32) return attention_launch<TYPE, 32>(ATT_ARGS);                                           \
  return PHOTON_ERR_UNSUPPORTED;

#define ATT_ARGS q, q_stride, out, out_stride, k_cache, v_cache, block_table, max_pages, token_seq, \
                 positions, T_, n_q, n_kv, d, page_size, num_pages, window, scale, err, stream

// window <= 0: all keys.  Strides in elements.  The cache holds [num_pages][n_kv][page_size][d].
PHOTON_API int photon_paged_attention(const void* q, long q_stride, void* out, long out_stride, int dtype,
                                      const void* k_cache, const void* v_cache, const int* block_table,
                                      int max_pages, const int* token_seq, const int* positions, int T_,
                                      int n_q, int n_kv, int d, int page_size, int num_pages, int window,
                                      float scale, int* err, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (n_kv <= 0 || n_q % n_kv || d <= 0 || page_size <= 0) return PHOTON_ERR_ARGUMENT;
  const int G = n_q / n_kv;
  const int ppt = (G * d + ATT_THREADS - 1) / ATT_THREADS;
  if (n_kv > 65535) return PHOTON_ERR_UNSUPPORTED;
  if (dtype == PHOTON_BF16) { ATT_DISPATCH(bf16) }
  ATT_DISPATCH(float)
}
