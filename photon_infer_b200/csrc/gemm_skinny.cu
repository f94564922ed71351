// Matrix product for few rows (decode steps): y[M, N] = x[M, K] * W[N, K]^T in bfloat16
// with 32-bit accumulation, M up to 64.  The weight matrix is streamed once from HBM
// with 16-byte loads that bypass L1; the product runs on the tensor cores with the
// roles swapped: 16 output features are the M side of mma.m16n8k16 and 8 tokens its N
// side, so no tensor-core work is wasted on padding a handful of tokens to 64 rows.
//
// A block owns 16 output features (32 with the SwiGLU epilogue: the gate rows and the
// matching up rows) and splits its share of K over its warps.  When the matrix has too
// few rows to fill the GPU, K is also split over up to 8 blocks per row tile: each
// block writes its sums to a scratch buffer in global memory and takes a ticket; the
// block that draws the last ticket adds all shares in rank order (so the result does
// not depend on timing), runs the epilogue and resets the ticket.  (A thread-block
// cluster with the shares in distributed shared memory was measured slower here: the
// cluster launch itself cost more than the scratch round trip.)  Epilogues:
//   EPI_BF16   y as bfloat16
//   EPI_F32    y as float (logits)
//   EPI_SWIGLU W is [2I, K] (gate rows, then up rows); y[M, I] = silu(gate) * up
//
// The k index inside a 32-wide block is permuted the same way for both operands (a
// lane's 8 consecutive elements feed two mma steps), which leaves the sum unchanged
// and lets every lane fetch its fragment with one 16-byte load.
//
// Same contract as the reference's product (include/photon/ops/kernels/
// matmul_kernel.hpp:104-129): W is [out, in] row-major, no bias.  The reference's own
// decode product is an INT8 GEMV on CUDA cores (src/ops/kernels/cuda/
// matmul_gemv_quant.cu:69-132).
#include "common.cuh"
#include <math.h>

#define SK_WARPS 8
#define SK_THREADS (SK_WARPS * 32)
#define EPI_BF16 0
#define EPI_F32 1
#define EPI_SWIGLU 2

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 r;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

// x is written by the kernel before this one, which may still be running when this kernel starts
// (programmatic dependent launch): it is read with ordinary loads after the wait, never through
// the read-only path.
__device__ __forceinline__ uint4 ld_plain16(const void* p) {
  uint4 r;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MT: token tiles of 8.  RT: row tiles of 16 per block (1, or 2 for SwiGLU: gate, up).
// UB: 1 doubles the loads a warp keeps in flight (for grids too small to hide latency by occupancy).
// Registers are capped for the large-grid variant, where 68 instead of 64 would cost the fourth resident
// block per SM (measured: the output head at 88 us instead of 84 us); the others are left to the compiler.
// NW: warps of a block, 8 or 16.  Sixteen split a long K inside one block (their sums meet in shared memory)
// where eight would need a second block and the hand-over through global memory.
template <int MT, int EPI, int UB, int NW = SK_WARPS>
__global__ void __launch_bounds__(NW * 32, (MT == 1 && UB == 0 && EPI != EPI_SWIGLU) ? 4 : 0)
skinny_gemm_kernel(const bf16* __restrict__ x, long ldx, const bf16* __restrict__ W, long ldw,
                   void* __restrict__ out, long ldo, int M, int N, int K, int I,
                   float* __restrict__ scratch, int* __restrict__ tickets) {
  constexpr int RT = (EPI == EPI_SWIGLU) ? 2 : 1;
  __shared__ float red[NW][RT * MT * 4 * 32];
  __shared__ int is_last;
  const int ks = gridDim.x;                        // blocks that share these rows and split K
  const int krank = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int n0 = blockIdx.y * 16;
  const int rows_total = (EPI == EPI_SWIGLU) ? I : N;

  // rows this lane loads: g and g + 8 of each row tile (clamped; masked at the store)
  const bf16* wrow[RT][2];
#pragma unroll
  for (int r = 0; r < RT; ++r)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int row = n0 + g + 8 * h;
      if (row >= rows_total) row = rows_total - 1;
      if (EPI == EPI_SWIGLU && r == 1) row += I;
      wrow[r][h] = W + (size_t)row * ldw;
    }
  const bf16* xrow[MT];
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    int tok = t * 8 + g;
    if (tok >= M) tok = M - 1;
    xrow[t] = x + (size_t)tok * ldx;
  }

  float acc[RT][MT][4];
#pragma unroll
  for (int r = 0; r < RT; ++r)
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[r][t][i] = 0.f;

  // k blocks of 32, dealt to the warps round-robin; a lane covers elements [c*8, c*8+8) of a block
  const int all_blocks = (K + 31) >> 5;
  const int per_rank = (all_blocks + ks - 1) / ks;
  const int kb0 = krank * per_rank;
  const int nblocks = min(all_blocks, kb0 + per_rank);
  constexpr int UNROLL = ((RT * MT <= 2) ? 4 : (RT * MT <= 4 ? 2 : 1)) * ((UB && RT * MT <= 1) ? 2 : 1);
  const int full_blocks = min(nblocks, K >> 5);      // k blocks that lie wholly inside K
  int kb = kb0 + warp;
  // The weights do not depend on the kernel before this one: their first loads are issued, then the
  // kernel waits for its predecessor (whose output is x), so the wait overlaps the memory latency.
  bool waited = false;
  // whole rounds: every load is issued before the first product, no predicates
  for (; kb + (UNROLL - 1) * NW < full_blocks; kb += NW * UNROLL) {
    uint4 wa[UNROLL][RT][2], xb[UNROLL][MT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (kb + u * NW) * 32 + c * 8;
#pragma unroll
      for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int h = 0; h < 2; ++h) wa[u][r][h] = ld_stream16(wrow[r][h] + k);
    }
    if (!waited) { pdl_wait(); waited = true; }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (kb + u * NW) * 32 + c * 8;
#pragma unroll
      for (int t = 0; t < MT; ++t)
        xb[u][t] = UB ? ld_plain16(xrow[t] + k) : __ldg(reinterpret_cast<const uint4*>(xrow[t] + k));
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          mma16816(acc[r][t], wa[u][r][0].x, wa[u][r][1].x, wa[u][r][0].y, wa[u][r][1].y, xb[u][t].x, xb[u][t].y);
          mma16816(acc[r][t], wa[u][r][0].z, wa[u][r][1].z, wa[u][r][0].w, wa[u][r][1].w, xb[u][t].z, xb[u][t].w);
        }
  }
  // what is left of this warp's blocks, one at a time; the last block of K may be partial
  for (; kb < nblocks; kb += NW) {
    const int k = kb * 32 + c * 8;
    const bool ok = k < K;                               // K is a multiple of 8
    uint4 wa[RT][2], xb[MT];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
      for (int h = 0; h < 2; ++h) wa[r][h] = ok ? ld_stream16(wrow[r][h] + k) : make_uint4(0, 0, 0, 0);
    if (!waited) { pdl_wait(); waited = true; }
#pragma unroll
    for (int t = 0; t < MT; ++t)
      xb[t] = !ok ? make_uint4(0, 0, 0, 0)
                  : (UB ? ld_plain16(xrow[t] + k) : __ldg(reinterpret_cast<const uint4*>(xrow[t] + k)));
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        mma16816(acc[r][t], wa[r][0].x, wa[r][1].x, wa[r][0].y, wa[r][1].y, xb[t].x, xb[t].y);
        mma16816(acc[r][t], wa[r][0].z, wa[r][1].z, wa[r][0].w, wa[r][1].w, xb[t].z, xb[t].w);
      }
  }

  if (!waited) pdl_wait();
  // The next kernel may be scheduled once every block has come this far (not earlier: its blocks would
  // take the places of blocks of this grid that have not started yet).
  pdl_launch_dependents();
  // add the warps' partial sums in warp order
#pragma unroll
  for (int r = 0; r < RT; ++r)
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) red[warp][((r * MT + t) * 4 + i) * 32 + lane] = acc[r][t][i];
  __syncthreads();
  // thread e of the block owns element (r, t, i, lane) = e of RT*MT*4*32; for SwiGLU r is folded
  constexpr int PER = MT * 4 * 32;
  float* shares = scratch + (size_t)blockIdx.y * ks * (RT * PER);
  if (ks > 1) {
    for (int e = threadIdx.x; e < RT * PER; e += (NW * 32)) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) v += red[w][e];
      __stcg(shares + (size_t)krank * (RT * PER) + e, v);
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = (atomicAdd(tickets + blockIdx.y, 1) == ks - 1);
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (threadIdx.x == 0) tickets[blockIdx.y] = 0;  // ready for the next launch
  }
  for (int e = threadIdx.x; e < PER; e += (NW * 32)) {
    const int ln = e & 31, i = (e >> 5) & 3, t = e >> 7;
    float v0 = 0.f, v1 = 0.f;
    if (ks > 1) {
      for (int r = 0; r < ks; ++r) {
        v0 += __ldcg(shares + (size_t)r * (RT * PER) + e);
        if (RT == 2) v1 += __ldcg(shares + (size_t)r * (RT * PER) + PER + e);
      }
    } else {
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        v0 += red[w][e];
        if (RT == 2) v1 += red[w][PER + e];
      }
    }
    const int row = n0 + (ln >> 2) + ((i & 2) ? 8 : 0);          // output feature
    const int tok = t * 8 + (ln & 3) * 2 + (i & 1);              // token
    if (row >= rows_total || tok >= M) continue;
    if (EPI == EPI_SWIGLU) {
      const float s = v0 / (1.0f + __expf(-v0));
      ((bf16*)out)[(size_t)tok * ldo + row] = __float2bfloat16_rn(s * v1);
    } else if (EPI == EPI_F32) {
      ((float*)out)[(size_t)tok * ldo + row] = v0;
    } else {
      ((bf16*)out)[(size_t)tok * ldo + row] = __float2bfloat16_rn(v0);
    }
  }
}

template <int EPI>
static int skinny_launch(const void* x, long ldx, const void* W, long ldw, void* out, long ldo, int M, int N,
                         int K, float* scratch, long scratch_floats, int* tickets, int num_tickets,
                         cudaStream_t stream) {
  const int I = N / 2;
  const int rows = (EPI == EPI_SWIGLU) ? I : N;
  const int row_blocks = (rows + 15) / 16;
  if (row_blocks > 65535) return PHOTON_ERR_UNSUPPORTED;
  const int mt = (M + 7) / 8;
  const int mt_pad = mt <= 1 ? 1 : (mt <= 2 ? 2 : (mt <= 4 ? 4 : 8));
  const int rt = (EPI == EPI_SWIGLU) ? 2 : 1;
  const int sms = photon_sm_count();
  const bool small_grid = row_blocks <= 4 * sms;
  const int unroll = ((rt * mt_pad <= 2) ? 4 : (rt * mt_pad <= 4 ? 2 : 1)) * ((small_grid && rt * mt_pad <= 1) ? 2 : 1);
  // split K over blocks only where a warp would need more than two rounds of loads and the row tiles alone leave
  // SMs without a block: the hand-over through global memory costs about as much as one round, and with a block
  // on every SM it only adds to it (measured at 8 rows: 4,096 x 14,336 in 22.9 us unsplit against 32.2 us in
  // halves, 3,072 x 8,192 in 13.3 against 16.8 us)
  // one block per SM or fewer: sixteen warps per block share K (2,048 x 2,048: 4.7 us against 5.1 us with eight)
  const bool wide = mt <= 1 && small_grid && EPI != EPI_SWIGLU && row_blocks <= sms && K >= 2048;
  const int warps = wide ? 16 : SK_WARPS;
  const int per_warp = ((K + 31) / 32 + warps - 1) / warps;
  int ks = 1;
  while (ks < 8 && per_warp > 2 * unroll * ks && row_blocks * ks < sms) ks *= 2;
  if (scratch == nullptr || tickets == nullptr || row_blocks > num_tickets) ks = 1;
  while (ks > 1 && (long)row_blocks * ks * rt * mt_pad * 128 > scratch_floats) ks /= 2;
  dim3 grid(ks, row_blocks);
  int st = 0;
  // The UB = 0 variants (large grids) read x through the read-only path and are launched fully serialised.
#define SK_GO(MT_)                                                                                          \
  (skinny_gemm_kernel<MT_, EPI, 0><<<grid, SK_THREADS, 0, stream>>>((const bf16*)x, ldx, (const bf16*)W, ldw, \
                                                                    out, ldo, M, N, K, I, scratch, tickets), \
   st = launch_status())
  if (wide)
    st = launch_pdl(skinny_gemm_kernel<1, EPI, 1, 16>, grid, dim3(16 * 32), 0, stream, (const bf16*)x, ldx,
                    (const bf16*)W, ldw, out, ldo, M, N, K, I, scratch, tickets);
  else if (mt <= 1 && small_grid && EPI != EPI_SWIGLU)
    st = launch_pdl(skinny_gemm_kernel<1, EPI, 1>, grid, dim3(SK_THREADS), 0, stream, (const bf16*)x, ldx,
                    (const bf16*)W, ldw, out, ldo, M, N, K, I, scratch, tickets);
  else if (mt <= 1) SK_GO(1);
  else if (mt <= 2) SK_GO(2);
  else if (mt <= 4) SK_GO(4);
  else if (mt <= 8) {
    if constexpr (EPI != EPI_SWIGLU) SK_GO(8);
    else return PHOTON_ERR_UNSUPPORTED;
  } else return PHOTON_ERR_UNSUPPORTED;
#undef SK_GO
  return st;
}

// epilogue: 0 bfloat16, 1 float, 2 SwiGLU (W holds 2I rows, out is [M, I]).
// Needs K % 8 == 0 and 16-byte aligned rows of x and W; M <= 64 (32 with SwiGLU).
// scratch (float) and tickets (int, all zero between launches) serve the split of K over blocks;
// without them K is not split.  Launches that share them must not overlap on the device.
PHOTON_API int photon_skinny_gemm(const void* x, long ldx, const void* W, long ldw, void* out, long ldo, int M,
                                  int N, int K, int epilogue, float* scratch, long scratch_floats, int* tickets,
                                  int num_tickets, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ((uintptr_t)x & 15) || ((uintptr_t)W & 15))
    return PHOTON_ERR_UNSUPPORTED;
  if (epilogue == EPI_SWIGLU && (N & 1)) return PHOTON_ERR_ARGUMENT;
  switch (epilogue) {
    case EPI_BF16: return skinny_launch<EPI_BF16>(x, ldx, W, ldw, out, ldo, M, N, K, scratch, scratch_floats, tickets, num_tickets, stream);
    case EPI_F32: return skinny_launch<EPI_F32>(x, ldx, W, ldw, out, ldo, M, N, K, scratch, scratch_floats, tickets, num_tickets, stream);
    case EPI_SWIGLU: return skinny_launch<EPI_SWIGLU>(x, ldx, W, ldw, out, ldo, M, N, K, scratch, scratch_floats, tickets, num_tickets, stream);
  }
  return PHOTON_ERR_ARGUMENT;
}
