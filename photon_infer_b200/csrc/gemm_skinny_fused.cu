// Decode-step products with their neighbours fused in (up to 8 rows, bfloat16):
//
//   prologue  x = residual_in + delta (32-bit), written to residual_out by the first block;
//             RMSNorm folded into the product: the kernel multiplies x * w_norm (rounded to
//             bfloat16) into W and scales the result by 1/sqrt(mean(x^2) + eps) at the end,
//             so the normed activations are never written
//   product   y[M, N] = xw[M, K] * W[N, K]^T as in gemm_skinny.cu: mma.m16n8k16 with swapped
//             roles, weights streamed once with 16-byte loads that bypass L1, K split over
//             the 8 warps of a block, partial sums added in warp order
//   epilogue  EPI_BF16    y as bfloat16
//             EPI_SWIGLU  W = [gate rows; up rows], y[M, I] = silu(gate) * up
//             EPI_QKV     W = [q; k; v] rows with rotation partners as neighbours: q and k are
//                         rotated (angle pos * inv_freq[pair], sine and cosine in 32-bit), q goes
//                         to `out`, k and v go straight into the paged cache at slot_mapping
//
// Replaces, for a decode step, the kernels add_rmsnorm + product (+ rope_kv_write): three
// launches fewer per layer.  Formulas: include/photon/ops/kernels/rmsnorm_kernel.hpp:71-86,
// rope_kernel.hpp:143-165, swiglu_kernel.hpp:67-76; cache layout of rope_kv.cu.
#include "common.cuh"
#include <math.h>

#define SF_WARPS 8
#define SF_THREADS (SF_WARPS * 32)
#define SF_UNROLL 4
#define EPI_BF16 0
#define EPI_SWIGLU 2
#define EPI_QKV 3

struct SkinnyFusedArgs {
  const float* res_in; float* res_out; const bf16* delta;       // [M, K]; delta may be null
  const void* norm_w; int norm_w_bf16; float eps;               // [K]
  const bf16* W; long ldw;                                      // [N, K]
  bf16* out; long ldo;                                          // [M, N] (EPI_SWIGLU: [M, N/2]; EPI_QKV: q columns only used)
  int M, N, K;
  // EPI_QKV
  const int* positions; const float* inv_freq; const int* slot_mapping;
  bf16* k_cache; bf16* v_cache;
  int n_q, n_kv, d, page_size; long num_slots;
  int* err;
};

__device__ __forceinline__ uint4 sf_ld_stream16(const void* p) {
  uint4 r;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
__device__ __forceinline__ void sf_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t sf_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int EPI>
__global__ void __launch_bounds__(SF_THREADS, 2)
skinny_fused_kernel(const SkinnyFusedArgs A) {
  constexpr int RT = (EPI == EPI_SWIGLU) ? 2 : 1;
  __shared__ float red[SF_WARPS][RT * 4 * 32];
  __shared__ float ssq[SF_WARPS][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int I = A.N / 2;
  const int rows_total = (EPI == EPI_SWIGLU) ? I : A.N;
  const bool writer = blockIdx.x == 0 && A.res_out != nullptr;

  const bf16* wrow[RT][2];
#pragma unroll
  for (int r = 0; r < RT; ++r)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int row = n0 + g + 8 * h;
      if (row >= rows_total) row = rows_total - 1;
      if (EPI == EPI_SWIGLU && r == 1) row += I;
      wrow[r][h] = A.W + (size_t)row * A.ldw;
    }
  const int tok = g < A.M ? g : A.M - 1;                    // the token whose x this lane loads
  const float* rrow = A.res_in + (size_t)tok * A.K;
  const bf16* drow = A.delta ? A.delta + (size_t)tok * A.K : nullptr;
  float* orow = writer ? A.res_out + (size_t)tok * A.K : nullptr;

  float acc[RT][4];
#pragma unroll
  for (int r = 0; r < RT; ++r) { acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f; }
  float ss = 0.f;

  // one k block of 32: this lane's 8 elements of x -> bfloat16 fragment of x * w_norm
  auto make_x = [&](int k, bool ok) -> uint4 {
    if (!ok) return make_uint4(0, 0, 0, 0);
    const float4 r0 = *reinterpret_cast<const float4*>(rrow + k);
    const float4 r1 = *reinterpret_cast<const float4*>(rrow + k + 4);
    float x[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
    if (drow) {
      const uint4 dv = *reinterpret_cast<const uint4*>(drow + k);
      const __nv_bfloat162* dp = reinterpret_cast<const __nv_bfloat162*>(&dv);
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(dp[i]); x[2 * i] += f.x; x[2 * i + 1] += f.y; }
    }
    if (writer && g < A.M) {
      *reinterpret_cast<float4*>(orow + k) = make_float4(x[0], x[1], x[2], x[3]);
      *reinterpret_cast<float4*>(orow + k + 4) = make_float4(x[4], x[5], x[6], x[7]);
    }
    float w[8];
    if (A.norm_w_bf16) {
      const uint4 wv = __ldg(reinterpret_cast<const uint4*>((const bf16*)A.norm_w + k));
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(wp[i]); w[2 * i] = f.x; w[2 * i + 1] = f.y; }
    } else {
      const float4 w0 = __ldg(reinterpret_cast<const float4*>((const float*)A.norm_w + k));
      const float4 w1 = __ldg(reinterpret_cast<const float4*>((const float*)A.norm_w + k + 4));
      w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w; w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
    uint4 o;
    o.x = sf_pack(x[0] * w[0], x[1] * w[1]); o.y = sf_pack(x[2] * w[2], x[3] * w[3]);
    o.z = sf_pack(x[4] * w[4], x[5] * w[5]); o.w = sf_pack(x[6] * w[6], x[7] * w[7]);
    return o;
  };

  const int nblocks = (A.K + 31) >> 5;
  const int full_blocks = A.K >> 5;
  int kb = warp;
  bool waited = false;
  for (; kb + (SF_UNROLL - 1) * SF_WARPS < full_blocks; kb += SF_WARPS * SF_UNROLL) {
    uint4 wa[SF_UNROLL][RT][2], xb[SF_UNROLL];
#pragma unroll
    for (int u = 0; u < SF_UNROLL; ++u) {
      const int k = (kb + u * SF_WARPS) * 32 + c * 8;
#pragma unroll
      for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int h = 0; h < 2; ++h) wa[u][r][h] = sf_ld_stream16(wrow[r][h] + k);
    }
    if (!waited) { pdl_wait(); waited = true; }
#pragma unroll
    for (int u = 0; u < SF_UNROLL; ++u) xb[u] = make_x((kb + u * SF_WARPS) * 32 + c * 8, true);
#pragma unroll
    for (int u = 0; u < SF_UNROLL; ++u)
#pragma unroll
      for (int r = 0; r < RT; ++r) {
        sf_mma(acc[r], wa[u][r][0].x, wa[u][r][1].x, wa[u][r][0].y, wa[u][r][1].y, xb[u].x, xb[u].y);
        sf_mma(acc[r], wa[u][r][0].z, wa[u][r][1].z, wa[u][r][0].w, wa[u][r][1].w, xb[u].z, xb[u].w);
      }
  }
  for (; kb < nblocks; kb += SF_WARPS) {
    const int k = kb * 32 + c * 8;
    const bool ok = k < A.K;
    uint4 wa[RT][2];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
      for (int h = 0; h < 2; ++h) wa[r][h] = ok ? sf_ld_stream16(wrow[r][h] + k) : make_uint4(0, 0, 0, 0);
    if (!waited) { pdl_wait(); waited = true; }
    const uint4 xb = make_x(k, ok);
#pragma unroll
    for (int r = 0; r < RT; ++r) {
      sf_mma(acc[r], wa[r][0].x, wa[r][1].x, wa[r][0].y, wa[r][1].y, xb.x, xb.y);
      sf_mma(acc[r], wa[r][0].z, wa[r][1].z, wa[r][0].w, wa[r][1].w, xb.z, xb.w);
    }
  }
  if (!waited) pdl_wait();
  pdl_launch_dependents();                         // after the main loop: see gemm_skinny.cu

  // sum of squares of token g: over the four lanes that share it, then over the warps
  ss += __shfl_xor_sync(0xffffffffu, ss, 1);
  ss += __shfl_xor_sync(0xffffffffu, ss, 2);
  if (c == 0) ssq[warp][g] = ss;
#pragma unroll
  for (int r = 0; r < RT; ++r)
#pragma unroll
    for (int i = 0; i < 4; ++i) red[warp][(r * 4 + i) * 32 + lane] = acc[r][i];
  __syncthreads();

  for (int e = threadIdx.x; e < 128; e += SF_THREADS) {      // warps 0..3, all lanes
    const int ln = e & 31, i = e >> 5;
    float v0 = 0.f, v1 = 0.f;
#pragma unroll
    for (int w = 0; w < SF_WARPS; ++w) {
      v0 += red[w][e];
      if (RT == 2) v1 += red[w][128 + e];
    }
    const int row = n0 + (ln >> 2) + ((i & 2) ? 8 : 0);       // output feature
    const int t = (ln & 3) * 2 + (i & 1);                     // token
    float s2 = 0.f;
#pragma unroll
    for (int w = 0; w < SF_WARPS; ++w) s2 += ssq[w][t];
    const float inv = 1.0f / sqrtf(s2 / (float)A.K + A.eps);
    v0 *= inv; v1 *= inv;
    if (EPI == EPI_QKV) {
      // the partner feature (row ^ 1) sits in lane ln ^ 4 of the same warp
      const float other = __shfl_xor_sync(0xffffffffu, v0, 4);
      if (row >= rows_total || t >= A.M) continue;
      const int qk_rows = (A.n_q + A.n_kv) * A.d;
      float y = v0;
      if (row < qk_rows) {
        const int j = (row % A.d) >> 1;
        float sn, cs;
        sincosf((float)A.positions[t] * A.inv_freq[j], &sn, &cs);
        y = (row & 1) ? other * sn + v0 * cs : v0 * cs - other * sn;
      }
      const bf16 yb = __float2bfloat16_rn(y);
      if (row < A.n_q * A.d) {
        A.out[(size_t)t * A.ldo + row] = yb;
      } else {
        const long slot = A.slot_mapping[t];
        if (slot < 0 || slot >= A.num_slots) {
          if (slot != -1) report_error(A.err, PHOTON_DEV_BAD_SLOT, t, (int)slot, (int)A.num_slots);
          continue;
        }
        const bool is_k = row < qk_rows;
        const int r2 = row - (is_k ? A.n_q * A.d : qk_rows);
        const int h = r2 / A.d, dd = r2 - h * A.d;
        const long page = slot / A.page_size;
        const int off = (int)(slot - page * A.page_size);
        bf16* cache = is_k ? A.k_cache : A.v_cache;
        cache[(((size_t)page * A.n_kv + h) * A.page_size + off) * A.d + dd] = yb;
      }
    } else {
      if (row >= rows_total || t >= A.M) continue;
      if (EPI == EPI_SWIGLU) {
        const float s = v0 / (1.0f + __expf(-v0));
        A.out[(size_t)t * A.ldo + row] = __float2bfloat16_rn(s * v1);
      } else {
        A.out[(size_t)t * A.ldo + row] = __float2bfloat16_rn(v0);
      }
    }
  }
}

// epilogue: 0 bfloat16, 2 SwiGLU, 3 QKV with rotation and cache write.
// M <= 8, K a multiple of 8, 16-byte aligned rows; the q/k rows of W must have rotation partners as
// neighbours (feature 2j with 2j + 1) and head_dim even; n_q * d, n_kv * d multiples of 2.
PHOTON_API int photon_skinny_fused(const float* res_in, float* res_out, const void* delta, const void* norm_w,
                                   int norm_w_dtype, float eps, const void* W, long ldw, void* out, long ldo, int M,
                                   int N, int K, int epilogue, const int* positions, const float* inv_freq,
                                   const int* slot_mapping, void* k_cache, void* v_cache, int n_q, int n_kv, int d,
                                   int page_size, long num_slots, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 8 || K <= 0 || (K & 7) || (ldw & 7) || ((uintptr_t)W & 15) || ((uintptr_t)res_in & 15) ||
      ((uintptr_t)res_out & 15) || ((uintptr_t)delta & 15) || ((uintptr_t)norm_w & 15))
    return PHOTON_ERR_UNSUPPORTED;
  if (epilogue == EPI_SWIGLU && (N & 1)) return PHOTON_ERR_ARGUMENT;
  if (epilogue == EPI_QKV && ((d & 1) || N != (n_q + 2 * n_kv) * d || positions == nullptr || inv_freq == nullptr ||
                              slot_mapping == nullptr || k_cache == nullptr || v_cache == nullptr))
    return PHOTON_ERR_ARGUMENT;
  SkinnyFusedArgs A;
  A.res_in = res_in; A.res_out = res_out; A.delta = (const bf16*)delta; A.norm_w = norm_w;
  A.norm_w_bf16 = (norm_w_dtype == PHOTON_BF16); A.eps = eps; A.W = (const bf16*)W; A.ldw = ldw;
  A.out = (bf16*)out; A.ldo = ldo; A.M = M; A.N = N; A.K = K;
  A.positions = positions; A.inv_freq = inv_freq; A.slot_mapping = slot_mapping;
  A.k_cache = (bf16*)k_cache; A.v_cache = (bf16*)v_cache; A.n_q = n_q; A.n_kv = n_kv; A.d = d;
  A.page_size = page_size; A.num_slots = num_slots; A.err = err;
  const int rows = (epilogue == EPI_SWIGLU) ? N / 2 : N;
  dim3 grid((rows + 15) / 16);
  switch (epilogue) {
    case EPI_BF16: return launch_pdl(skinny_fused_kernel<EPI_BF16>, grid, dim3(SF_THREADS), 0, stream, A);
    case EPI_SWIGLU: return launch_pdl(skinny_fused_kernel<EPI_SWIGLU>, grid, dim3(SF_THREADS), 0, stream, A);
    case EPI_QKV: return launch_pdl(skinny_fused_kernel<EPI_QKV>, grid, dim3(SF_THREADS), 0, stream, A);
  }
  return PHOTON_ERR_ARGUMENT;
}
