// Matrix product for many rows on pairs of SMs: C[M, N] = A[M, K] * W[N, K]^T, bfloat16 in,
// 32-bit accumulation in tensor memory, tiles of 256 x 256 computed by two blocks of a
// cluster with tcgen05.mma.cta_group::2.
//
// Same scheme as gemm_tc.cu (TMA into a ring of stages, one issuing thread, two accumulators,
// tcgen05.ld epilogue, persistent blocks), with these differences:
//   * the two blocks of a cluster own rows m0 .. m0 + 127 and m0 + 128 .. m0 + 255 of a tile;
//     each loads its own 128 x 64 tile of A and HALF of the 256 x 64 tile of W per stage (block
//     0 the first 128 rows of W, block 1 the other 128).  The product instruction of block 0
//     reads A and W from both blocks' shared memory and writes both blocks' tensor memory, so
//     every SM fetches 32 KB per 64 of K instead of 48 KB: the operand traffic from L2 that
//     bounds the one-block kernel drops by a third.
//   * the TMA loads of both blocks complete on block 0's "full" barrier (cta_group::2 form of
//     the copy; the barrier address with the peer bit cleared); tcgen05.commit with a multicast
//     mask frees a stage, and publishes an accumulator, in both blocks at once; the epilogue
//     warps of block 1 arrive on block 0's "accumulator free" barrier through the cluster
//     address space.
//   * SwiGLU epilogue: block 0 holds the 128 gate rows and block 1 the matching 128 up rows, so
//     accumulator columns 0..127 are gate and 128..255 up, as in the one-block kernel.
//
// Every wait is bounded by elapsed cycles; a wait that runs out raises the block's abort flag,
// records PHOTON_DEV_WAIT_TIMEOUT and every role leaves its loop.  The two blocks of a cluster
// meet at a cluster barrier before the tensor memory is freed, so neither exits while the other
// may still address its shared or tensor memory.
#include "tcgen05.cuh"

#define T2_BM 128                     // rows per block (256 per cluster)
#define T2_BN 256
#define T2_BK 64
#ifndef T2_STAGES
#define T2_STAGES 6
#endif
#define T2_THREADS 192                // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue
#define T2_A_BYTES (T2_BM * T2_BK * 2)
#define T2_B_BYTES ((T2_BN / 2) * T2_BK * 2)      // this block's half of the W tile
#define T2_STAGE_BYTES (T2_A_BYTES + T2_B_BYTES)
#define T2_SMEM_BYTES (T2_STAGES * T2_STAGE_BYTES + 1024 + 256)
#define T2_PEER_MASK 0xFEFFFFFFu      // clears the bit of a shared::cluster address that names the odd block of a pair
#ifndef T2_WAIT_CYCLES
#define T2_WAIT_CYCLES (4000000000LL) // about two seconds
#endif

#define T2_EPI_BF16 0
#define T2_EPI_F32 1
#define T2_EPI_SWIGLU 2
#define T2_EPI_QKV 3                  // rows of q | k | v: q and k rotated, q to `out`, k and v into the paged cache

// What the QKV epilogue needs beside the product (formulas: include/photon/ops/kernels/rope_kernel.hpp:54-84 for
// the rotation of neighbouring pairs, src/ops/kernels/cuda/paged_kv_write.cu:26-77 for the cache write).
struct T2Qkv {
  const int* positions;               // [M]
  const int* slot_mapping;            // [M] slot of the token in the paged cache, -1: not stored
  const float* inv_freq;              // [d / 2]
  const float2* table;                // (cos, sin) [table_positions, d / 2] or null
  bf16* k_cache; bf16* v_cache;       // [pages, n_kv, page_size, d]
  int table_positions, n_q, n_kv, d, page_size;
  long num_slots;
};

__device__ __forceinline__ bool t2_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const long long t0 = clock64();
  for (uint32_t i = 0;; ++i) {
    if (tc_mbar_try(bar, parity)) return true;
    if ((i & 63) == 63) {
      if (*abort_flag) return false;
      if (clock64() - t0 > T2_WAIT_CYCLES) { *abort_flag = 1; return false; }
    }
  }
}
__device__ __forceinline__ uint32_t t2_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void t2_cluster_sync() {
  asm volatile("barrier.cluster.arrive.aligned;\nbarrier.cluster.wait.aligned;" ::: "memory");
}
// The copy of a pair: the bytes are counted on block 0's barrier whichever block issues it.
__device__ __forceinline__ void t2_tma_load(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(tc_smem(dst)), "l"(map), "r"(tc_smem(bar) & T2_PEER_MASK), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void t2_mma(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}"
               ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// Arrives, once the products issued so far are done, on the barrier at this address in both blocks of the pair.
__device__ __forceinline__ void t2_commit_both(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(tc_smem(bar)), "h"((unsigned short)3) : "memory");
}
// One arrival on block 0's barrier at this address, from either block.
__device__ __forceinline__ void t2_arrive_block0(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(tc_smem(bar) & T2_PEER_MASK) : "memory");
}

template <int EPI>
__global__ void __launch_bounds__(T2_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                void* __restrict__ out, long ldo, int M, int N, int K, int I, int tiles_n, int num_tiles, int* err,
                const T2Qkv Q) {
  extern __shared__ unsigned char t2_dyn[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)t2_dyn + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + T2_STAGES * T2_STAGE_BYTES);
  uint64_t* full = bars;                          // [T2_STAGES] used in block 0: both blocks' TMA -> MMA
  uint64_t* empty = bars + T2_STAGES;             // [T2_STAGES] in each block: MMA -> that block's TMA
  uint64_t* acc_ready = bars + 2 * T2_STAGES;     // [2] in each block: MMA -> that block's epilogue
  uint64_t* acc_free = bars + 2 * T2_STAGES + 2;  // [2] used in block 0: both blocks' epilogues -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * T2_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = t2_cta_rank();            // 0 or 1 inside the pair
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_kb = (K + T2_BK - 1) / T2_BK;
  constexpr int TILE_COLS = (EPI == T2_EPI_SWIGLU) ? T2_BN / 2 : T2_BN;      // output columns of a tile

  if (threadIdx.x == 0) {
    for (int s = 0; s < T2_STAGES; ++s) { tc_mbar_init(&full[s], 1); tc_mbar_init(&empty[s], 1); }
    for (int b2 = 0; b2 < 2; ++b2) { tc_mbar_init(&acc_ready[b2], 1); tc_mbar_init(&acc_free[b2], 8); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    // the same warp of both blocks allocates: two accumulators of T2_BN columns in each block's tensor memory
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(tmem_slot)), "n"(2 * T2_BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  t2_cluster_sync();                              // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                                     // A is the output of the kernel before

  if (warp == 0) {
    // ---------------- producer (one lane in each block): this block's rows of A and its half of the W tile
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int m0 = (tile / tiles_n) * (2 * T2_BM) + (int)rank * T2_BM, n0 = (tile % tiles_n) * TILE_COLS;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % T2_STAGES;
          if (!t2_wait(&empty[s], ((it / T2_STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
          unsigned char* a_dst = tiles + s * T2_STAGE_BYTES;
          unsigned char* b_dst = a_dst + T2_A_BYTES;
          if (rank == 0) tc_mbar_expect_tx(&full[s], 2 * T2_STAGE_BYTES);     // both blocks' bytes
          t2_tma_load(a_dst, &map_a, kb * T2_BK, m0, &full[s]);
          if (EPI == T2_EPI_SWIGLU) t2_tma_load(b_dst, &map_w, kb * T2_BK, (rank == 0 ? 0 : I) + n0, &full[s]);
          else t2_tma_load(b_dst, &map_w, kb * T2_BK, n0 + (int)rank * (T2_BN / 2), &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: one lane of block 0 issues for the pair
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = tc_idesc(2 * T2_BM, T2_BN);
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
        const int buf = local & 1;
        if (!t2_wait(&acc_free[buf], ((local >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * T2_BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % T2_STAGES;
          if (!t2_wait(&full[s], (it / T2_STAGES) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = tc_smem(tiles + s * T2_STAGE_BYTES);
          const uint32_t b_addr = a_addr + T2_A_BYTES;
#pragma unroll
          for (int k = 0; k < T2_BK / 16; ++k)
            t2_mma(d_tmem, tc_desc(a_addr + k * 32), tc_desc(b_addr + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          t2_commit_both(&empty[s]);                // both blocks may refill the stage once these products have read it
        }
        if (ok) t2_commit_both(&acc_ready[buf]);
      }
      pdl_launch_dependents();
    }
  } else {
    // ---------------- epilogue: warps 2..5 of each block own TMEM lanes 32 * (warp % 4) .. + 31 of that block
    const int quad = warp & 3;
    const int ncols = (EPI == T2_EPI_SWIGLU) ? I : N;
    int local = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local) {
      const int buf = local & 1;
      if (!t2_wait(&acc_ready[buf], (local >> 1) & 1, abort_flag)) break;
      tc_fence_after();
      const int m0 = (tile / tiles_n) * (2 * T2_BM) + (int)rank * T2_BM, n0 = (tile % tiles_n) * TILE_COLS;
      const int row = m0 + quad * 32 + lane;
      const uint32_t lane_addr = tmem_base + buf * T2_BN + ((uint32_t)(quad * 32) << 16);
      // QKV epilogue: the token's position and its place in the cache, once per tile
      int pos = 0;
      long cache_row = -1;                          // (page * n_kv) * page_size + offset in the page, or -1
      if (EPI == T2_EPI_QKV && row < M) {
        pos = Q.positions[row];
        const long slot = Q.slot_mapping[row];
        if (slot >= Q.num_slots || slot < -1) report_error(err, PHOTON_DEV_BAD_SLOT, row, (int)slot, (int)Q.num_slots);
        else if (slot >= 0) {
          const long page = slot / Q.page_size;
          cache_row = page * Q.n_kv * Q.page_size + (slot - page * Q.page_size);
        }
      }
      // (cos, sin) of the token's 16 pairs at head offsets j0 = 0 and 32 (mod 64): with heads of 64 every other
      // chunk of a tile asks for the same 16, so they are fetched once per tile, 16 bytes at a time
      float4 rot_a[8], rot_b[8];
      int rot_a_j0 = -1, rot_b_j0 = -1;
#pragma unroll 1
      for (int c = 0; c < TILE_COLS; c += 32) {
        uint32_t v[32], u[32];
        tc_ld32(lane_addr + c, v);
        if (EPI == T2_EPI_SWIGLU) tc_ld32(lane_addr + T2_BN / 2 + c, u);
        if (row < M) {
          const int col0 = n0 + c;
          if (EPI == T2_EPI_QKV) {
            if (col0 < N) {                           // N is a multiple of 32 here: the chunk is inside one head
              const int qd = Q.n_q * Q.d, kd = Q.n_kv * Q.d, half = Q.d >> 1;
              const int which = col0 < qd ? 0 : (col0 < qd + kd ? 1 : 2);
              const int local = col0 - (which == 0 ? 0 : (which == 1 ? qd : qd + kd));
              const int h = local / Q.d, j0 = local - h * Q.d;
              float y[32];
              if (which < 2) {
                // two sets of registers, chosen by a branch (indexing them would put them in local memory)
                auto rotate = [&](float4 (&rot)[8], int& have_j0) {
                  if (have_j0 != j0) {
                    have_j0 = j0;
                    if (Q.table != nullptr && pos < Q.table_positions) {
                      const float4* trow = reinterpret_cast<const float4*>(Q.table + (size_t)pos * half + (j0 >> 1));
#pragma unroll
                      for (int i = 0; i < 8; ++i) rot[i] = trow[i];           // 16-byte aligned: j0 is a multiple of 32
                    } else {
#pragma unroll
                      for (int i = 0; i < 8; ++i) {
                        float4 t4;
                        sincosf((float)pos * Q.inv_freq[(j0 >> 1) + 2 * i], &t4.y, &t4.x);
                        sincosf((float)pos * Q.inv_freq[(j0 >> 1) + 2 * i + 1], &t4.w, &t4.z);
                        rot[i] = t4;
                      }
                    }
                  }
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    const float4 t4 = rot[i];                                 // (cos, sin) of two pairs
                    const float a0 = __uint_as_float(v[4 * i]), a1 = __uint_as_float(v[4 * i + 1]);
                    const float b0 = __uint_as_float(v[4 * i + 2]), b1 = __uint_as_float(v[4 * i + 3]);
                    y[4 * i] = a0 * t4.x - a1 * t4.y;
                    y[4 * i + 1] = a0 * t4.y + a1 * t4.x;
                    y[4 * i + 2] = b0 * t4.z - b1 * t4.w;
                    y[4 * i + 3] = b0 * t4.w + b1 * t4.z;
                  }
                };
                if ((j0 >> 5) & 1) rotate(rot_b, rot_b_j0);
                else rotate(rot_a, rot_a_j0);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) y[j] = __uint_as_float(v[j]);
              }
              bf16* dst = nullptr;
              if (which == 0) dst = (bf16*)out + (size_t)row * ldo + col0;
              else if (cache_row >= 0)
                dst = (which == 1 ? Q.k_cache : Q.v_cache) + ((size_t)cache_row + (size_t)h * Q.page_size) * Q.d + j0;
              if (dst != nullptr) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  uint4 pk;
                  __nv_bfloat162 p0 = __floats2bfloat162_rn(y[j], y[j + 1]), p1 = __floats2bfloat162_rn(y[j + 2], y[j + 3]);
                  __nv_bfloat162 p2 = __floats2bfloat162_rn(y[j + 4], y[j + 5]), p3 = __floats2bfloat162_rn(y[j + 6], y[j + 7]);
                  pk.x = *reinterpret_cast<uint32_t*>(&p0); pk.y = *reinterpret_cast<uint32_t*>(&p1);
                  pk.z = *reinterpret_cast<uint32_t*>(&p2); pk.w = *reinterpret_cast<uint32_t*>(&p3);
                  *reinterpret_cast<uint4*>(dst + j) = pk;
                }
              }
            }
          } else if (EPI == T2_EPI_F32) {
            float* dst = (float*)out + (size_t)row * ldo + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j) if (col0 + j < ncols) dst[j] = __uint_as_float(v[j]);
          } else {
            bf16* dst = (bf16*)out + (size_t)row * ldo + col0;
            float y[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float g = __uint_as_float(v[j]);
              y[j] = (EPI == T2_EPI_SWIGLU) ? __fdividef(g, 1.0f + __expf(-g)) * __uint_as_float(u[j]) : g;
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
      // this warp has read its lanes: one arrival per warp, from both blocks, on block 0's barrier
      tc_fence_before();
      __syncwarp();
      if (lane == 0) t2_arrive_block0(&acc_free[buf]);
    }
  }
  // ---------------- teardown: both blocks meet, then the allocating warps free the tensor memory
  if (*abort_flag) {
    // copies this block issued may still be writing its shared memory (their barrier is in block 0, where this
    // block cannot wait): give them 200,000 cycles, far more than a copy takes
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {}
  }
  tc_fence_before();
  __syncthreads();
  t2_cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(2 * T2_BN) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag) report_error(err, PHOTON_DEV_WAIT_TIMEOUT, blockIdx.x, 0, 0);
}

// ---------------------------------------------------------------- host side
static int t2_launch(const void* x, long ldx, const void* W, long ldw, void* out, long ldo, int M, int N, int K,
                     int epilogue, const T2Qkv& Q, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ((uintptr_t)x & 15) || ((uintptr_t)W & 15))
    return PHOTON_ERR_UNSUPPORTED;
  if (epilogue == T2_EPI_SWIGLU && (N & 1)) return PHOTON_ERR_ARGUMENT;
  if (epilogue < 0 || epilogue > 3) return PHOTON_ERR_ARGUMENT;
  const int I = N / 2;
  CUtensorMap map_a, map_w;
  int st = make_map(&map_a, x, M, K, ldx, T2_BM);
  if (st != 0) return st;
  st = make_map(&map_w, W, N, K, ldw, T2_BN / 2);
  if (st != 0) return st;
  const int out_cols = epilogue == T2_EPI_SWIGLU ? I : N;
  const int tile_cols = epilogue == T2_EPI_SWIGLU ? T2_BN / 2 : T2_BN;
  const int tiles_n = (out_cols + tile_cols - 1) / tile_cols;
  const long total = (long)tiles_n * ((M + 2 * T2_BM - 1) / (2 * T2_BM));
  if (total > 0x7fffffff) return PHOTON_ERR_UNSUPPORTED;
  const int num_tiles = (int)total;
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0) num_sms = 148;
  }
  const int pairs = num_tiles < num_sms / 2 ? num_tiles : num_sms / 2;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e[4];
    e[0] = cudaFuncSetAttribute(gemm_tc2_kernel<T2_EPI_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM_BYTES);
    e[1] = cudaFuncSetAttribute(gemm_tc2_kernel<T2_EPI_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM_BYTES);
    e[2] = cudaFuncSetAttribute(gemm_tc2_kernel<T2_EPI_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM_BYTES);
    e[3] = cudaFuncSetAttribute(gemm_tc2_kernel<T2_EPI_QKV>, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM_BYTES);
    for (int i = 0; i < 4; ++i) if (e[i] != cudaSuccess) return (int)e[i];
    attr_done = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(T2_THREADS); cfg.dynamicSmemBytes = T2_SMEM_BYTES; cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = photon_pdl_enabled(stream) ? 2 : 1;
  cudaError_t e;
#define T2_GO(EPI_) cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<EPI_>, map_a, map_w, out, ldo, M, N, K, I, tiles_n, num_tiles, err, Q)
  switch (epilogue) {
    case T2_EPI_BF16: e = T2_GO(T2_EPI_BF16); break;
    case T2_EPI_F32: e = T2_GO(T2_EPI_F32); break;
    case T2_EPI_SWIGLU: e = T2_GO(T2_EPI_SWIGLU); break;
    default: e = T2_GO(T2_EPI_QKV); break;
  }
#undef T2_GO
  if (e != cudaSuccess) return (int)e;
  return launch_status();
}

// epilogue: 0 bfloat16, 1 float, 2 SwiGLU (W holds 2I rows, out is [M, I]).  Same requirements as photon_gemm_tc.
PHOTON_API int photon_gemm_tc2(const void* x, long ldx, const void* W, long ldw, void* out, long ldo, int M, int N,
                               int K, int epilogue, int* err, cudaStream_t stream) {
  if (epilogue < 0 || epilogue > 2) return PHOTON_ERR_ARGUMENT;
  T2Qkv Q = {};
  return t2_launch(x, ldx, W, ldw, out, ldo, M, N, K, epilogue, Q, err, stream);
}

// The q/k/v product of a step with rotation and cache write in the epilogue: W [(n_q + 2 n_kv) d, K] holds the
// rows of q, then k, then v, rotation partners of q and k as neighbours; q_out [M, n_q d] gets the rotated
// queries, the rotated keys and the values go to slot_mapping[row] of the paged cache ([pages, n_kv, page_size,
// d]; slot -1: not stored).  d must be a multiple of 32.  table (may be null): (cos, sin) for positions below
// table_positions, else they are computed in place.
PHOTON_API int photon_gemm_tc2_qkv(const void* x, long ldx, const void* W, long ldw, void* q_out, long ldo, int M,
                                   int K, const int* positions, const int* slot_mapping, const float* inv_freq,
                                   const void* table, int table_positions, void* k_cache, void* v_cache, int n_q,
                                   int n_kv, int d, int page_size, long num_slots, int* err, cudaStream_t stream) {
  if (n_q <= 0 || n_kv <= 0 || d <= 0 || (d & 31) || page_size <= 0) return PHOTON_ERR_UNSUPPORTED;
  if (positions == nullptr || slot_mapping == nullptr || inv_freq == nullptr || k_cache == nullptr || v_cache == nullptr)
    return PHOTON_ERR_ARGUMENT;
  if (((uintptr_t)q_out & 15) || (ldo & 7) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15)) return PHOTON_ERR_ARGUMENT;
  T2Qkv Q;
  Q.positions = positions; Q.slot_mapping = slot_mapping; Q.inv_freq = inv_freq; Q.table = (const float2*)table;
  Q.table_positions = table != nullptr ? table_positions : 0;
  Q.k_cache = (bf16*)k_cache; Q.v_cache = (bf16*)v_cache; Q.n_q = n_q; Q.n_kv = n_kv; Q.d = d; Q.page_size = page_size;
  Q.num_slots = num_slots;
  const long N = (long)(n_q + 2 * n_kv) * d;
  if (N > 0x7fffffff) return PHOTON_ERR_UNSUPPORTED;
  return t2_launch(x, ldx, W, ldw, q_out, ldo, M, (int)N, K, T2_EPI_QKV, Q, err, stream);
}
