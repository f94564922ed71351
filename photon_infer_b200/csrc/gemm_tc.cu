// Matrix product for many rows (prompt portions) on the fifth-generation tensor cores:
// C[M, N] = A[M, K] * W[N, K]^T, bfloat16 in, 32-bit accumulation in tensor memory.
//
//   * operands: TMA (cp.async.bulk.tensor.2d, 128-byte swizzle) brings 128 x 64 tiles of A
//     and 256 x 64 tiles of W into a ring of shared-memory stages; completion by mbarrier
//   * product: one elected thread issues tcgen05.mma (M = 128, N = 256, K = 16 per
//     instruction, cta_group::1); two accumulators of 256 TMEM columns alternate
//   * epilogue: four warps read an accumulator back with tcgen05.ld (one TMEM lane =
//     one output row per thread) and write bfloat16, float, or silu(gate) * up, while
//     the products of the block's next tile are already being issued
//   * one block per SM walks the tiles (persistent)
//
// With the SwiGLU epilogue W is [2I, K] (gate rows, then up rows): a stage gets the 128
// gate rows and the matching 128 up rows as the two halves of its 256-row tile, so the
// gate and up values of the same 128 features sit side by side in the accumulator and
// no activation of width 2I is ever written.
//
// Same contract as the reference's product (include/photon/ops/kernels/matmul_kernel.hpp:
// 104-129: W [out, in] row-major, no bias); the reference's engine calls cublasSgemm on
// dequantised weights here (src/ops/kernels/cuda/matmul_dequant_cached.cu:193-207).
//
// Every wait on an mbarrier is bounded.  When one runs out the block raises an abort flag
// that all roles poll, records PHOTON_DEV_WAIT_TIMEOUT, waits (bounded) for the copies it
// has in flight, frees its tensor memory and returns.
#include "tcgen05.cuh"

#define TC_BM 128
#ifndef TC_BN
#define TC_BN 256
#endif
#define TC_BK 64                      // 64 bf16 = 128 bytes = one swizzle row
#ifndef TC_STAGES
#define TC_STAGES 4
#endif
#define TC_UMMA_K 16
#define TC_THREADS 192                // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue
#define TC_A_BYTES (TC_BM * TC_BK * 2)
#define TC_B_BYTES (TC_BN * TC_BK * 2)
#define TC_STAGE_BYTES (TC_A_BYTES + TC_B_BYTES)
#define TC_SMEM_BYTES (TC_STAGES * TC_STAGE_BYTES + 1024 + 256)

#define TC_EPI_BF16 0
#define TC_EPI_F32 1
#define TC_EPI_SWIGLU 2

// Persistent: a block walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...; tiles are numbered with the
// N index fastest.  Two accumulators of TC_BN columns alternate, so the epilogue of one tile runs while
// the products of the next are issued.
template <int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               void* __restrict__ out, long ldo, int M, int N, int K, int I, int tiles_n, int num_tiles, int* err) {
  extern __shared__ unsigned char tc_dyn[];
  // tiles need 1024-byte alignment for the 128-byte swizzle
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)tc_dyn + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + TC_STAGES * TC_STAGE_BYTES);
  uint64_t* full = bars;                          // [TC_STAGES] TMA -> MMA
  uint64_t* empty = bars + TC_STAGES;             // [TC_STAGES] MMA -> TMA
  uint64_t* acc_ready = bars + 2 * TC_STAGES;     // [2] MMA -> epilogue
  uint64_t* acc_free = bars + 2 * TC_STAGES + 2;  // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TC_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (K + TC_BK - 1) / TC_BK;
  constexpr int TILE_COLS = (EPI == TC_EPI_SWIGLU) ? TC_BN / 2 : TC_BN;      // output columns of a tile

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) { tc_mbar_init(&full[s], 1); tc_mbar_init(&empty[s], 1); }
    for (int b2 = 0; b2 < 2; ++b2) { tc_mbar_init(&acc_ready[b2], 1); tc_mbar_init(&acc_free[b2], 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    // the whole warp allocates two accumulators of TC_BN columns; the address lands in shared memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(tmem_slot)), "n"(2 * TC_BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                                     // A is the output of the kernel before; the set-up above overlapped its tail

  if (warp == 0) {
    // ---------------- producer: one lane issues the TMA loads, the ring runs on across tiles
    if (lane == 0) {
      int it = 0;                                   // k blocks issued so far
      bool ok = true;
#ifdef TC_TEST_NO_LOADS
      ok = false;                                   // test build: nothing is ever loaded, so the waits below run out
#endif
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile / tiles_n) * TC_BM, n0 = (tile % tiles_n) * TILE_COLS;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % TC_STAGES;
          if (!tc_wait(&empty[s], ((it / TC_STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
          unsigned char* a_dst = tiles + s * TC_STAGE_BYTES;
          unsigned char* b_dst = a_dst + TC_A_BYTES;
          tc_mbar_expect_tx(&full[s], TC_STAGE_BYTES);
          tc_tma_load(a_dst, &map_a, kb * TC_BK, m0, &full[s]);
          if (EPI == TC_EPI_SWIGLU) {
            tc_tma_load(b_dst, &map_w, kb * TC_BK, n0, &full[s]);                        // 128 gate rows
            tc_tma_load(b_dst + TC_B_BYTES / 2, &map_w, kb * TC_BK, I + n0, &full[s]);   // the matching up rows
          } else {
            tc_tma_load(b_dst, &map_w, kb * TC_BK, n0, &full[s]);
          }
        }
      }
      if (*abort_flag) {
        // copies already issued still write into this block's shared memory: wait for them, bounded
        for (int j = (it > TC_STAGES ? it - TC_STAGES : 0); j < it; ++j)
          for (uint32_t i = 0; i < TC_WAIT_LIMIT && !tc_mbar_try(&full[j % TC_STAGES], (j / TC_STAGES) & 1); ++i) {}
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: one lane
    if (lane == 0) {
      const uint32_t idesc = tc_idesc(TC_BM, TC_BN);
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        // the epilogue must have drained this accumulator (two tiles ago)
        if (!tc_wait(&acc_free[buf], ((local >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + buf * TC_BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % TC_STAGES;
          if (!tc_wait(&full[s], (it / TC_STAGES) & 1, abort_flag)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = tc_smem(tiles + s * TC_STAGE_BYTES);
          const uint32_t b_addr = a_addr + TC_A_BYTES;
#pragma unroll
          for (int k = 0; k < TC_BK / TC_UMMA_K; ++k) {
            // 16 elements of K = 32 bytes further inside the swizzled 128-byte rows
            tc_mma(d_tmem, tc_desc(a_addr + k * 32), tc_desc(b_addr + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty[s]);                     // the stage is free once these products have read it
        }
        if (ok) tc_commit(&acc_ready[buf]);         // the accumulator is complete once all products are done
      }
      pdl_launch_dependents();                      // all products of this block are issued
    }
  } else {
    // ---------------- epilogue: warps 2..5 own TMEM lanes 32 * (warp % 4) .. + 31
    const int quad = warp & 3;
    const int ncols = (EPI == TC_EPI_SWIGLU) ? I : N;
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      if (!tc_wait(&acc_ready[buf], (local >> 1) & 1, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int m0 = (tile / tiles_n) * TC_BM, n0 = (tile % tiles_n) * TILE_COLS;
      const int row = m0 + quad * 32 + lane;
      const uint32_t lane_addr = tmem_base + buf * TC_BN + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < TILE_COLS; c += 32) {
        uint32_t v[32], u[32];
        tc_ld32(lane_addr + c, v);                 // all lanes take part, also those of rows beyond M
        if (EPI == TC_EPI_SWIGLU) tc_ld32(lane_addr + TC_BN / 2 + c, u);
        if (row < M) {
          const int col0 = n0 + c;
          if (EPI == TC_EPI_F32) {
            float* dst = (float*)out + (size_t)row * ldo + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j) if (col0 + j < ncols) dst[j] = __uint_as_float(v[j]);
          } else {
            bf16* dst = (bf16*)out + (size_t)row * ldo + col0;
            float y[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float g = __uint_as_float(v[j]);
              y[j] = (EPI == TC_EPI_SWIGLU) ? __fdividef(g, 1.0f + __expf(-g)) * __uint_as_float(u[j]) : g;
            }
            if (col0 + 32 <= ncols && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 pk;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(y[j], y[j + 1]), p1 = __floats2bfloat162_rn(y[j + 2], y[j + 3]);
                __nv_bfloat162 p2 = __floats2bfloat162_rn(y[j + 4], y[j + 5]), p3 = __floats2bfloat162_rn(y[j + 6], y[j + 7]);
                pk.x = *reinterpret_cast<uint32_t*>(&p0); pk.y = *reinterpret_cast<uint32_t*>(&p1);
                pk.z = *reinterpret_cast<uint32_t*>(&p2); pk.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(dst + j) = pk;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) if (col0 + j < ncols) dst[j] = __float2bfloat16_rn(y[j]);
            }
          }
        }
      }
      // this warp has read its lanes of the accumulator: one arrival per warp frees it for the tile after next
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem(&acc_free[buf])) : "memory");
    }
  }
  // ---------------- teardown: everyone meets, the allocating warp frees the tensor memory
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(2 * TC_BN) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag) report_error(err, PHOTON_DEV_WAIT_TIMEOUT, blockIdx.x, 0, 0);
}

// ---------------------------------------------------------------- host side
// epilogue: 0 bfloat16, 1 float, 2 SwiGLU (W holds 2I rows, out is [M, I]).
// Needs 16-byte aligned bases and row strides that are a multiple of 8 elements (TMA), K a multiple of 8.
PHOTON_API int photon_gemm_tc(const void* x, long ldx, const void* W, long ldw, void* out, long ldo, int M, int N,
                              int K, int epilogue, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ((uintptr_t)x & 15) || ((uintptr_t)W & 15))
    return PHOTON_ERR_UNSUPPORTED;
  if (epilogue == TC_EPI_SWIGLU && (N & 1)) return PHOTON_ERR_ARGUMENT;
  const int I = N / 2;
  CUtensorMap map_a, map_w;
  int st = make_map(&map_a, x, M, K, ldx, TC_BM);
  if (st != 0) return st;
  st = make_map(&map_w, W, N, K, ldw, epilogue == TC_EPI_SWIGLU ? TC_BN / 2 : TC_BN);
  if (st != 0) return st;
  const int out_cols = epilogue == TC_EPI_SWIGLU ? I : N;
  const int tile_cols = epilogue == TC_EPI_SWIGLU ? TC_BN / 2 : TC_BN;
  const int tiles_n = (out_cols + tile_cols - 1) / tile_cols;
  const long total = (long)tiles_n * ((M + TC_BM - 1) / TC_BM);
  if (total > 0x7fffffff) return PHOTON_ERR_UNSUPPORTED;
  const int num_tiles = (int)total;
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0) num_sms = 148;
  }
  dim3 grid(num_tiles < num_sms ? num_tiles : num_sms);
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e0 = cudaFuncSetAttribute(gemm_tc_kernel<TC_EPI_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
    cudaError_t e1 = cudaFuncSetAttribute(gemm_tc_kernel<TC_EPI_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
    cudaError_t e2 = cudaFuncSetAttribute(gemm_tc_kernel<TC_EPI_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
    if (e0 != cudaSuccess) return (int)e0;
    if (e1 != cudaSuccess) return (int)e1;
    if (e2 != cudaSuccess) return (int)e2;
    attr_done = true;
  }
  switch (epilogue) {
    case TC_EPI_BF16:
      return launch_pdl(gemm_tc_kernel<TC_EPI_BF16>, grid, dim3(TC_THREADS), (size_t)TC_SMEM_BYTES, stream, map_a, map_w, out, ldo, M, N, K, I, tiles_n, num_tiles, err);
    case TC_EPI_F32:
      return launch_pdl(gemm_tc_kernel<TC_EPI_F32>, grid, dim3(TC_THREADS), (size_t)TC_SMEM_BYTES, stream, map_a, map_w, out, ldo, M, N, K, I, tiles_n, num_tiles, err);
    case TC_EPI_SWIGLU:
      return launch_pdl(gemm_tc_kernel<TC_EPI_SWIGLU>, grid, dim3(TC_THREADS), (size_t)TC_SMEM_BYTES, stream, map_a, map_w, out, ldo, M, N, K, I, tiles_n, num_tiles, err);
    default:
      return PHOTON_ERR_ARGUMENT;
  }
  return launch_status();
}
