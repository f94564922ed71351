// Sampling on the device: first-maximum argmax and temperature sampling by inverse
// CDF.  One block per row of 32-bit logits.
//
// Argmax: src/ops/kernels/cuda/sampling_kernel.cu:36-138 and src/arch/llama_model.cpp:
// 304-328 (the earliest index wins a tie).  Temperature: demo/llama_infer.cpp:78-101,
// p_i = exp((l_i - max) / T) / sum, the first i whose running sum reaches u; there it
// runs on the CPU with rand(), here u is given per row by the caller (a counter-based
// generator on the host), so a request's tokens do not depend on the batch.
#include "common.cuh"
#include <math.h>

#define SAMP_THREADS 1024

__device__ __forceinline__ void argmax_combine(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

__device__ int block_argmax(const float* row, int V, float* out_max) {
  __shared__ float sv[32];
  __shared__ int si[32];
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_combine(best, bi, ov, oi);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nwarp = (blockDim.x + 31) >> 5;
    best = lane < nwarp ? sv[lane] : -INFINITY;
    bi = lane < nwarp ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      argmax_combine(best, bi, ov, oi);
    }
    if (lane == 0) { sv[0] = best; si[0] = bi; }
  }
  __syncthreads();
  if (out_max) *out_max = sv[0];
  const int r = si[0];
  __syncthreads();
  return r == 0x7fffffff ? 0 : r;
}

// temperature[r] <= 0: greedy.  Else inverse-CDF sampling with u[r] in [0, 1).
// Each thread owns one contiguous span of the row, so the running sum is taken in index
// order: span sums first, then a scan over the 1024 spans, then inside the chosen span.
__global__ void __launch_bounds__(SAMP_THREADS)
sample_kernel(const float* __restrict__ logits, long ld, const float* __restrict__ temperature,
              const float* __restrict__ u, int* __restrict__ out, int V) {
  __shared__ float span_sum[SAMP_THREADS];
  __shared__ int chosen;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * ld;
  float mx;
  const int am = block_argmax(row, V, &mx);
  const float temp = temperature ? temperature[r] : 0.f;
  if (!(temp > 0.f)) {
    if (threadIdx.x == 0) out[r] = am;
    return;
  }
  const int span = (V + SAMP_THREADS - 1) / SAMP_THREADS;
  const int lo = threadIdx.x * span;
  const int hi = min(V, lo + span);
  float s = 0.f;
  for (int i = lo; i < hi; ++i) s += expf((row[i] - mx) / temp);
  span_sum[threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int i = 0; i < SAMP_THREADS; ++i) total += span_sum[i];
    const float target = u[r] * total;       // first i with cum_i / total >= u
    float cum = 0.f;
    int c = SAMP_THREADS - 1;
    for (int i = 0; i < SAMP_THREADS; ++i) {
      if (cum + span_sum[i] >= target && span_sum[i] > 0.f) { c = i; break; }
      cum += span_sum[i];
    }
    // walk inside the span
    const int l2 = c * span, h2 = min(V, l2 + span);
    int pick = -1;
    for (int i = l2; i < h2; ++i) {
      cum += expf((row[i] - mx) / temp);
      if (cum >= target) { pick = i; break; }
    }
    if (pick < 0) {
      // rounding left the total below the target: the last index with a non-zero probability
      pick = am;
      for (int i = V - 1; i >= 0; --i) if (expf((row[i] - mx) / temp) > 0.f) { pick = i; break; }
    }
    chosen = pick;
    out[r] = chosen;
  }
}

// ---------------------------------------------------------------- two passes for long rows
// Pass 1: the row is cut into SAMP_CHUNKS spans; block (chunk, row) finds the span's maximum, its first
// index and, for temperature rows, the sum of exp((l - span max) / T).  Pass 2: one block per row merges
// the spans in index order and, for temperature rows, walks the one span the target falls into.
#define SAMP_CHUNKS 32
#define SAMP_P1_THREADS 256

__global__ void __launch_bounds__(SAMP_P1_THREADS)
sample_pass1_kernel(const float* __restrict__ logits, long ld, const float* __restrict__ temperature,
                    float* __restrict__ part, int V) {
  __shared__ float red[32];
  const int r = blockIdx.y, c = blockIdx.x;
  const float* row = logits + (size_t)r * ld;
  const int span = (V + SAMP_CHUNKS - 1) / SAMP_CHUNKS;
  const int lo = c * span, hi = min(V, lo + span);
  float mx;
  const int am = hi > lo ? lo + block_argmax(row + lo, hi - lo, &mx) : 0;
  if (hi <= lo) mx = -INFINITY;
  const float temp = temperature ? temperature[r] : 0.f;
  float sum = 0.f;
  if (temp > 0.f && hi > lo) {
    float s = 0.f;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) s += expf((row[i] - mx) / temp);
    sum = block_sum(s, red);
  }
  if (threadIdx.x == 0) {
    float* p = part + ((size_t)r * SAMP_CHUNKS + c) * 4;
    p[0] = mx; p[1] = __int_as_float(am); p[2] = sum; p[3] = 0.f;
  }
}

__global__ void __launch_bounds__(SAMP_THREADS)
sample_pass2_kernel(const float* __restrict__ logits, long ld, const float* __restrict__ temperature,
                    const float* __restrict__ u, const float* __restrict__ part, int* __restrict__ out, int V) {
  __shared__ float span_sum[SAMP_THREADS];
  __shared__ int s_chunk;
  __shared__ float s_before, s_target, s_max;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * ld;
  const float* p = part + (size_t)r * SAMP_CHUNKS * 4;
  const float temp = temperature ? temperature[r] : 0.f;
  if (threadIdx.x == 0) {
    float M = -INFINITY; int am = 0;
    for (int c = 0; c < SAMP_CHUNKS; ++c) if (p[c * 4] > M) { M = p[c * 4]; am = __float_as_int(p[c * 4 + 1]); }
    s_max = M;
    s_chunk = -1;
    if (!(temp > 0.f)) {
      out[r] = am;
    } else {
      float total = 0.f;
      for (int c = 0; c < SAMP_CHUNKS; ++c) if (p[c * 4] != -INFINITY) total += p[c * 4 + 2] * expf((p[c * 4] - M) / temp);
      const float target = u[r] * total;
      float cum = 0.f; int pick = -1;
      for (int c = 0; c < SAMP_CHUNKS; ++c) {
        const float sc = p[c * 4] != -INFINITY ? p[c * 4 + 2] * expf((p[c * 4] - M) / temp) : 0.f;
        if (sc > 0.f && cum + sc >= target) { pick = c; break; }
        cum += sc;
      }
      if (pick < 0) {                                  // rounding left the total below the target
        for (int c = SAMP_CHUNKS - 1; c >= 0; --c) if (p[c * 4] != -INFINITY && p[c * 4 + 2] > 0.f) { pick = c; break; }
        cum = target;                                  // take the last element of that span with weight
      }
      s_chunk = pick; s_before = cum; s_target = target;
      out[r] = am;                                     // replaced below
    }
  }
  __syncthreads();
  if (s_chunk < 0) return;
  // inside the chosen span: every thread owns a contiguous piece, pieces are scanned in order
  const int span = (V + SAMP_CHUNKS - 1) / SAMP_CHUNKS;
  const int lo = s_chunk * span, hi = min(V, lo + span);
  const int piece = (hi - lo + SAMP_THREADS - 1) / SAMP_THREADS;
  const int plo = lo + threadIdx.x * piece, phi = min(hi, plo + piece);
  float s = 0.f;
  for (int i = plo; i < phi; ++i) s += expf((row[i] - s_max) / temp);
  span_sum[threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float cum = s_before;
    int t = -1;
    for (int i = 0; i < SAMP_THREADS; ++i) {
      if (span_sum[i] > 0.f && cum + span_sum[i] >= s_target) { t = i; break; }
      cum += span_sum[i];
    }
    int pick = -1;
    if (t >= 0) {
      const int l2 = lo + t * piece, h2 = min(hi, l2 + piece);
      for (int i = l2; i < h2; ++i) {
        cum += expf((row[i] - s_max) / temp);
        if (cum >= s_target) { pick = i; break; }
      }
      if (pick < 0) pick = h2 - 1;
    } else {
      for (int i = hi - 1; i >= lo; --i) if (expf((row[i] - s_max) / temp) > 0.f) { pick = i; break; }
    }
    if (pick >= 0) out[r] = pick;
  }
}

// scratch: float [rows * 32 * 4] for rows longer than 16384 (two passes); may be null, then one pass is used.
PHOTON_API int photon_sample(const float* logits, long ld, const float* temperature, const float* u, int* out,
                             int rows, int V, float* scratch, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V <= 0) return PHOTON_ERR_ARGUMENT;
  if (scratch != nullptr && V > 16384 && rows <= 65535) {
    dim3 g1(SAMP_CHUNKS, rows);
    sample_pass1_kernel<<<g1, SAMP_P1_THREADS, 0, stream>>>(logits, ld, temperature, scratch, V);
    int st = launch_status();
    if (st != 0) return st;
    sample_pass2_kernel<<<rows, SAMP_THREADS, 0, stream>>>(logits, ld, temperature, u, scratch, out, V);
    return launch_status();
  }
  sample_kernel<<<rows, SAMP_THREADS, 0, stream>>>(logits, ld, temperature, u, out, V);
  return launch_status();
}
