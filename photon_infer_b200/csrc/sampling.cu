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

PHOTON_API int photon_sample(const float* logits, long ld, const float* temperature, const float* u, int* out,
                             int rows, int V, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V <= 0) return PHOTON_ERR_ARGUMENT;
  sample_kernel<<<rows, SAMP_THREADS, 0, stream>>>(logits, ld, temperature, u, out, V);
  return launch_status();
}
