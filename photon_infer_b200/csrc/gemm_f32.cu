// True 32-bit matrix product for the float32 path: C[M,N] = A[M,K] * W[N,K]^T with
// plain FMA on the CUDA cores, no tensor-core mode of reduced precision.  Same
// contract as the reference's naive product (include/photon/ops/kernels/
// matmul_kernel.hpp:104-129: W is [out, in] row-major, no bias).
//
// Every output element is one chain of K fused multiply-adds in ascending k, so a
// row's result does not depend on M, on the tile it fell into or on the other rows:
// the float32 path gives identical bits for every way of cutting a request into steps.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

__global__ void __launch_bounds__(256)
sgemm_nt_kernel(const float* __restrict__ A, long lda, const float* __restrict__ W, long ldw,
                float* __restrict__ C, long ldc, int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4 x 4 outputs each
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k: thread loads 4 elements of A and of W
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int idx = tid + r * 256;                // 0..1023
      const int row = idx >> 4, kk = idx & 15;
      const int gm = m0 + row, gn = n0 + row, gk = k0 + kk;
      As[kk][row] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
      Ws[kk][row] = (gn < N && gk < K) ? W[(size_t)gn * ldw + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j];
    }
  }
}

PHOTON_API int photon_sgemm_nt(const float* A, long lda, const float* W, long ldw, float* C, long ldc,
                               int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return PHOTON_ERR_ARGUMENT;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return PHOTON_ERR_UNSUPPORTED;
  sgemm_nt_kernel<<<grid, 256, 0, stream>>>(A, lda, W, ldw, C, ldc, M, N, K);
  return launch_status();
}
