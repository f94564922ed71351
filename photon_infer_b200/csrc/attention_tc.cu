// Paged causal attention for prompt portions on the fifth-generation tensor cores
// (tcgen05, accumulators in tensor memory), bfloat16, head size 64 or 128.
//
// A block owns up to 128 query rows of one request that share a key/value head
// (row = token_in_step * GROUP + head_in_group, as in attention_flash.cu; floor(128 / GROUP)
// whole tokens) and walks the
// request's keys in tiles of 64 (AT_KT):
//   * warp 4 brings the rows of Q (one 3-D TMA box) and then the key and value tiles of the
//     paged cache (one TMA box per page part, the block table followed by the lanes of the
//     warp) into a ring of shared-memory stages, 128-byte swizzle;
//   * one thread of warp 5 issues S = Q K^T (tcgen05.mma, M 128, N 64) into one of two score
//     buffers in tensor memory, and O += P V (M 128, N = head size; V is read as it lies in
//     the cache, keys along the rows, through an MN-major descriptor);
//   * warps 0-3 own one row per thread: they read the scores with tcgen05.ld, keep the
//     running maximum and sum in 32-bit, write P = exp2(..) as bfloat16 back over the scores in
//     tensor memory (the second product takes its A operand from there), and rescale O in tensor memory only when
//     a row's maximum has grown by more than 2^8 since the last rescale (the sum and O stay
//     relative to the maximum in use, so the result is the same up to rounding).
// The scores of tile i + 1 are computed while the softmax of tile i runs.
//
// Formula: include/photon/ops/kernels/mha_kernel.hpp:188-229 (scores (q.k)/sqrt(d) for the
// keys up to the token's own position, softmax, weighted sum of values; head h uses
// key/value head h / (n_q/n_kv)), with an optional window.  The reference has no
// tensor-core attention (src/ops/kernels/cuda/paged_attention.cu:90-194).
//
// Keys beyond a row's position are masked by selection, so what their cache rows hold does not
// matter for the scores; their value rows are multiplied by P = 0, so the rows of the last tile
// that lie beyond the request's last key (not yet written, or left by an earlier owner of the
// page) are set to zero in shared memory before the product reads them.  Page parts wholly
// beyond the last key or before the window are not read at all (TMA zero fill).
//
// Every wait on an mbarrier is bounded.  When one runs out the block raises an abort flag
// that all roles poll, records PHOTON_DEV_WAIT_TIMEOUT, waits (bounded) for the copies it
// has in flight, frees its tensor memory and returns.
//
// Compiled per model with -DHEAD_DIM=<64|128>.
#include "tcgen05.cuh"
#include <math.h>

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
static_assert(HEAD_DIM == 64 || HEAD_DIM == 128, "head size of the tcgen05 attention");

#define AT_ROWS 128
// Keys per tile.  -DAT_KT=128 (heads of 64 only: two stages of such tiles leave room for two blocks per SM) halves the
// hand-overs per key, but tensor memory then holds ONE score buffer beside O, so the scores of the next tile wait
// for P V of this one: measured 47.5 us against 38.6 us at 2,048 tokens, 522 against 427 us at 8,192.
#ifndef AT_KT
#define AT_KT 64
#endif
static_assert(AT_KT == 64 || HEAD_DIM == 64, "tiles of 128 keys only at heads of 64");
static_assert(AT_KT == 64 || AT_KT == 128, "keys per tile");
#define AT_NBUF (AT_KT == 128 ? 1 : 2)             // score buffers in tensor memory (128 columns in all)
#ifndef AT_STAGES
#define AT_STAGES (HEAD_DIM * AT_KT == 64 * 64 ? 3 : 2)   // two blocks per SM either way (81 KB, or 97 KB at heads of 128)
#endif
#ifndef AT_BLOCKS_PER_SM
#define AT_BLOCKS_PER_SM 2
#endif
#define AT_THREADS 192                             // warps 0-3: softmax, warp 4: TMA, warp 5: MMA + TMEM
#define AT_DH (HEAD_DIM / 64)                      // 64-wide halves of the head dimension
#define AT_Q_BYTES (AT_ROWS * HEAD_DIM * 2)
#define AT_KV_BYTES (AT_KT * HEAD_DIM * 2)         // one K tile or one V tile
#define AT_HALF_BYTES (AT_KT * 128)                // one 64-wide half of a K or V tile
#ifndef AT_P_TMEM
#define AT_P_TMEM 1                                // 1: P stays in tensor memory (it takes the place of the scores it came from)
#endif
#define AT_P_BYTES (AT_P_TMEM ? 0 : AT_ROWS * AT_KT * 2)
static_assert(AT_P_TMEM || AT_KT == 64, "P in shared memory only with tiles of 64 keys");
#define AT_SMEM_BYTES (AT_Q_BYTES + AT_STAGES * 2 * AT_KV_BYTES + 2 * AT_P_BYTES + 1024 + 256)
#define AT_TMEM_COLS 256                           // scores 2 x 64 or 1 x 128 columns, O from column 128
#define AT_O_COL 128
#define AT_RESCALE_STEP 8.0f                       // log2 units a maximum may lag behind before O is rescaled

struct AttnTcParams {
  bf16* out; long out_stride;                      // [T, n_q * d]
  const int* block_table; int max_pages;           // [S, max_pages]
  const int* cu_tokens;                            // [S + 1]
  const int* positions;                            // [T]
  int n_kv, group, tile_rows, page_size, num_pages, box_rows, window, tiles_per_seq, total_rows;
  float scale_log2;
  int* err;
};

// D += A B with A in tensor memory (128 lanes x 8 columns of packed bfloat16 pairs per 16 of K), B in shared memory.
__device__ __forceinline__ void at_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ float at_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two 32-bit lanes per instruction (sm_100): d = a * b + c and d = a + b on pairs.
__device__ __forceinline__ void at_fma2(float& d0, float& d1, float a0, float a1, float b, float c) {
  asm("{\n.reg .b64 ra, rb, rc, rd;\nmov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %4};\nmov.b64 rc, {%5, %5};\n"
      "fma.rn.f32x2 rd, ra, rb, rc;\nmov.b64 {%0, %1}, rd;\n}"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void at_add2(float& d0, float& d1, float a0, float a1) {
  asm("{\n.reg .b64 ra, rd;\nmov.b64 ra, {%2, %3};\nmov.b64 rd, {%0, %1};\n"
      "add.rn.f32x2 rd, rd, ra;\nmov.b64 {%0, %1}, rd;\n}"
      : "+f"(d0), "+f"(d1) : "f"(a0), "f"(a1));
}
__device__ __forceinline__ float at_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint32_t at_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(AT_THREADS, AT_BLOCKS_PER_SM)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const AttnTcParams P) {
  // ---- which rows: uniform for the block, before anything is set up
  const int g = blockIdx.x;
  const int seq = blockIdx.y / P.tiles_per_seq;
  const int qtile = P.tiles_per_seq - 1 - (blockIdx.y - seq * P.tiles_per_seq);   // most keys first
  const int G = P.group;
  pdl_wait();                                      // q, the cache and the step's tables come from kernels before
  const int tok0 = P.cu_tokens[seq], ntok = P.cu_tokens[seq + 1] - tok0;
  const int rows = ntok * G;
  const int row0 = qtile * P.tile_rows;            // tile_rows: the largest multiple of GROUP up to 128
  if (rows <= 16 || row0 >= rows) return;          // few rows: the split-key kernel takes this request
  const int nrows = min(P.tile_rows, rows - row0);
  const int t_first = row0 / G, t_last = (row0 + nrows - 1) / G;
  const int pos_first = P.positions[tok0 + t_first], pos_last = P.positions[tok0 + t_last];
  const int key_lo = (P.window > 0 && pos_first - P.window + 1 > 0) ? pos_first - P.window + 1 : 0;
  const int tile_begin = key_lo / AT_KT;
  const int ntiles = pos_last / AT_KT + 1 - tile_begin;

  extern __shared__ unsigned char at_dyn[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)at_dyn + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = base;
  unsigned char* kv_s = q_s + AT_Q_BYTES;                              // AT_STAGES x (K tile | V tile)
  unsigned char* p_s = kv_s + AT_STAGES * 2 * AT_KV_BYTES;             // 2 x P
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + 2 * AT_P_BYTES);
  uint64_t* q_full = bars;                          // TMA -> MMA
  uint64_t* k_full = bars + 1;                      // [AT_STAGES] TMA -> MMA
  uint64_t* v_full = k_full + AT_STAGES;            // [AT_STAGES] TMA -> MMA
  uint64_t* kv_empty = v_full + AT_STAGES;          // [AT_STAGES] MMA -> TMA
  uint64_t* s_full = kv_empty + AT_STAGES;          // [2] MMA -> softmax
  uint64_t* p_full = s_full + 2;                    // [2] softmax -> MMA (one arrival per warp)
  uint64_t* pv_done = p_full + 2;                   // [2] MMA -> softmax: P buffer free, O up to date
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    tc_mbar_init(q_full, 1);
    for (int s = 0; s < AT_STAGES; ++s) { tc_mbar_init(&k_full[s], 1); tc_mbar_init(&v_full[s], 1); tc_mbar_init(&kv_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { tc_mbar_init(&s_full[b], 1); tc_mbar_init(&p_full[b], 4); tc_mbar_init(&pv_done[b], 1); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(tmem_slot)), "n"(AT_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ---------------- producer
    if (lane == 0) {
      tc_mbar_expect_tx(q_full, P.tile_rows * 128 * AT_DH);       // rows beyond tile_rows stay as they are: nobody uses them
#pragma unroll
      for (int h = 0; h < AT_DH; ++h)
        tc_tma_load3(q_s + h * (AT_ROWS * 128), &map_q, h * 64, g * G, tok0 + t_first, q_full);
    }
    const int* table = P.block_table + (size_t)seq * P.max_pages;
    const int boxes = AT_KT / P.box_rows;           // parts of a tile that may lie in different pages
    int issued = 0;
    for (int i = 0; i < ntiles; ++i) {
      const int s = i % AT_STAGES;
      // the page of this lane's part, looked up before the wait for a free stage
      int rowc = P.total_rows;                      // outside the map: the part is filled with zeros
      if (lane < boxes) {
        const int key = (tile_begin + i) * AT_KT + lane * P.box_rows;
        if (key <= pos_last && key + P.box_rows - 1 >= key_lo) {
          const int pidx = key / P.page_size, slot = key - pidx * P.page_size;
          const int page = table[pidx];
          if (page < 0 || page >= P.num_pages) report_error(P.err, PHOTON_DEV_BAD_PAGE, tok0, key, page);
          else rowc = (page * P.n_kv + g) * P.page_size + slot;
        }
      }
      int ok = 1;
      if (lane == 0) ok = tc_wait(&kv_empty[s], ((i / AT_STAGES) & 1) ^ 1, abort_flag) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane == 0) { tc_mbar_expect_tx(&k_full[s], AT_KV_BYTES); tc_mbar_expect_tx(&v_full[s], AT_KV_BYTES); }
      __syncwarp();
      if (lane < boxes) {
        unsigned char* kst = kv_s + s * 2 * AT_KV_BYTES + lane * P.box_rows * 128;
        unsigned char* vst = kst + AT_KV_BYTES;
#pragma unroll
        for (int h = 0; h < AT_DH; ++h) tc_tma_load(kst + h * AT_HALF_BYTES, &map_k, h * 64, rowc, &k_full[s]);
#pragma unroll
        for (int h = 0; h < AT_DH; ++h) tc_tma_load(vst + h * AT_HALF_BYTES, &map_v, h * 64, rowc, &v_full[s]);
      }
      issued = i + 1;
    }
    if (lane == 0 && *abort_flag) {
      // copies already issued still write into this block's shared memory: wait for them, bounded
      for (uint32_t w = 0; w < TC_WAIT_LIMIT && !tc_mbar_try(q_full, 0); ++w) {}
      for (int j = (issued > AT_STAGES ? issued - AT_STAGES : 0); j < issued; ++j) {
        for (uint32_t w = 0; w < TC_WAIT_LIMIT && !tc_mbar_try(&k_full[j % AT_STAGES], (j / AT_STAGES) & 1); ++w) {}
        for (uint32_t w = 0; w < TC_WAIT_LIMIT && !tc_mbar_try(&v_full[j % AT_STAGES], (j / AT_STAGES) & 1); ++w) {}
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = tc_idesc(AT_ROWS, AT_KT);
      const uint32_t idesc_o = tc_idesc(AT_ROWS, HEAD_DIM) | TC_IDESC_B_MN;
      const uint32_t q_addr = tc_smem(q_s);
      auto issue_scores = [&](int i) -> bool {
        const int s = i % AT_STAGES;
        if (!tc_wait(&k_full[s], (i / AT_STAGES) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t k_addr = tc_smem(kv_s + s * 2 * AT_KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < HEAD_DIM / 16; ++kk)
          tc_mma(tmem_base + (i % AT_NBUF) * AT_KT, tc_desc(q_addr + (kk >> 2) * (AT_ROWS * 128) + (kk & 3) * 32),
                 tc_desc(k_addr + (kk >> 2) * AT_HALF_BYTES + (kk & 3) * 32), idesc_s, kk > 0 ? 1u : 0u);
        tc_commit(&s_full[i % AT_NBUF]);
        return true;
      };
      bool ok = tc_wait(q_full, 0, abort_flag);
      if (ok) ok = issue_scores(0);
      for (int i = 0; i < ntiles && ok; ++i) {
        // two score buffers: the next tile's scores are issued before this tile's P V; one buffer (P lies where the
        // scores were): after it, and the tensor core runs them in the order of issue
        if (AT_NBUF == 2 && i + 1 < ntiles) { ok = issue_scores(i + 1); if (!ok) break; }
        const int s = i % AT_STAGES;
        if (!tc_wait(&p_full[i % AT_NBUF], (i / AT_NBUF) & 1, abort_flag)) { ok = false; break; }
        if (!tc_wait(&v_full[s], (i / AT_STAGES) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t p_addr = tc_smem(p_s + (i & 1) * AT_P_BYTES);
        const uint32_t v_addr = tc_smem(kv_s + s * 2 * AT_KV_BYTES + AT_KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < AT_KT / 16; ++kk) {  // 16 keys: two groups of 8 rows of V
          if (AT_P_TMEM)                           // P: 8 columns of packed pairs per 16 keys, where the tile's scores were
            at_mma_ts(tmem_base + AT_O_COL, tmem_base + (i % AT_NBUF) * AT_KT + kk * 8, tc_desc_mn(v_addr + kk * 2048, AT_HALF_BYTES, 1024),
                      idesc_o, (i > 0 || kk > 0) ? 1u : 0u);
          else                                     // P: 32 bytes along a row of the swizzled tile in shared memory
            tc_mma(tmem_base + AT_O_COL, tc_desc(p_addr + kk * 32), tc_desc_mn(v_addr + kk * 2048, AT_HALF_BYTES, 1024),
                   idesc_o, (i > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&kv_empty[s]);
        tc_commit(&pv_done[i % AT_NBUF]);
        if (AT_NBUF == 1 && i + 1 < ntiles) ok = issue_scores(i + 1);
      }
      pdl_launch_dependents();                      // all products of this block are issued
    }
  } else {
    // ---------------- softmax: thread = row
    const int r = threadIdx.x;                      // 0..127
    const int row = row0 + r;
    const bool valid = r < P.tile_rows && row < rows;
    const int pos = valid ? P.positions[tok0 + row / G] : -1;
    const int lo = (P.window > 0 && pos - P.window + 1 > 0) ? pos - P.window + 1 : 0;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
    const float c = P.scale_log2;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    // the warp goes on or gives up together: tcgen05.ld/st need all of its lanes
    auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, tc_wait(bar, parity, abort_flag) ? 1 : 0) != 0;
    };
    for (int i = 0; i < ntiles; ++i) {
      const int b = i % AT_NBUF;
      if (!wait_all(&s_full[b], (i / AT_NBUF) & 1)) { ok = false; break; }
      tc_fence_after();
      const int key_base = (tile_begin + i) * AT_KT;
      const bool masked = !(key_base + AT_KT - 1 <= pos && key_base >= lo);
      // 64 scores of this row: keys key_base + 64 * half ..; those the row may not see become -inf
      uint32_t sv[64];
      auto load64 = [&](int half) {
        tc_ld32_issue(lane_addr + b * AT_KT + half * 64, sv);
        tc_ld32_issue(lane_addr + b * AT_KT + half * 64 + 32, sv + 32);
        tc_ld_wait();
        if (masked) {
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            const int key = key_base + half * 64 + j;
            sv[j] = (key >= lo && key <= pos) ? sv[j] : 0xff800000u;       // -inf
          }
        }
      };
      // first pass: the row's maximum, four independent chains of three-input maxima
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
      for (int half = 0; half < AT_KT / 64; ++half) {
        load64(half);
#pragma unroll
        for (int j = 0; j < 64; j += 8) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            mx4[u] = at_max3(mx4[u], __uint_as_float(sv[j + 2 * u]), __uint_as_float(sv[j + 2 * u + 1]));
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // the maximum in use lags behind the true one by at most AT_RESCALE_STEP
      const float cand = fmaxf(m_used, mx * c);
      float factor = 1.f;
      const bool grow = cand > m_used + AT_RESCALE_STEP;          // also the first finite maximum
      if (grow) { factor = at_exp2(m_used - cand); m_used = cand; l *= factor; }
      const float sub = (m_used == -INFINITY) ? 0.f : m_used;
      // O rescale: the products of the tile before must have landed
      if (i > 0 && __any_sync(0xffffffffu, grow)) {
        if (!wait_all(&pv_done[(i - 1) % AT_NBUF], ((i - 1) / AT_NBUF) & 1)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int cc = 0; cc < HEAD_DIM; cc += 32) {
          uint32_t ov[32];
          tc_ld32(lane_addr + AT_O_COL + cc, ov);
#pragma unroll
          for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * factor);
          tc_st32(lane_addr + AT_O_COL + cc, ov);
        }
        tc_st_wait();
      }
      if (i == ntiles - 1 && pos_last - key_base + 1 < AT_KT) {
        // value rows beyond the request's last key: zeros instead of whatever the page holds
        const int nvalid = pos_last - key_base + 1, nzero = AT_KT - nvalid;
        const int s = i % AT_STAGES;
        if (!wait_all(&v_full[s], (i / AT_STAGES) & 1)) { ok = false; break; }
        unsigned char* vst = kv_s + s * 2 * AT_KV_BYTES + AT_KV_BYTES;
        for (int e = r; e < nzero * 8 * AT_DH; e += AT_ROWS) {
          const int half = e / (nzero * 8), rem = e - half * (nzero * 8);
          *reinterpret_cast<uint4*>(vst + half * AT_HALF_BYTES + (nvalid + (rem >> 3)) * 128 + ((rem & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> the tensor core's reads
      }
      // second pass: P = exp2(score * c - max in use), 64 keys at a time (tiles of 128 keys: read again from tensor
      // memory, so that a row's scores never need 128 registers)
      float sum8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      const float nsub = -sub;
#pragma unroll 1
      for (int half = 0; half < AT_KT / 64; ++half) {
        if (AT_KT > 64) load64(half);
        uint32_t pk[32];
#pragma unroll
        for (int j = 0; j < 64; j += 2) {
          float x0, x1;
          at_fma2(x0, x1, __uint_as_float(sv[j]), __uint_as_float(sv[j + 1]), c, nsub);
          const float p0 = at_exp2(x0), p1 = at_exp2(x1);
          at_add2(sum8[j & 6], sum8[(j & 6) + 1], p0, p1);
          pk[j >> 1] = at_pack(p0, p1);
        }
        if (AT_P_TMEM) {
          // P over the scores it came from: packed pairs, 32 columns per 64 keys.  With tiles of 128 keys the first
          // half's P covers scores already read, and the second half's scores (columns 64..127) are still whole.
          tc_st32(lane_addr + b * AT_KT + half * 32, pk);
        } else {
          // the P buffer is free once the products of tile i - 2 have read it
          if (i >= 2 && !wait_all(&pv_done[b], ((i - 2) >> 1) & 1)) { ok = false; break; }
          unsigned char* prow = p_s + b * AT_P_BYTES + r * 128;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            uint4 v4 = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
            *reinterpret_cast<uint4*>(prow + ((ch ^ (r & 7)) << 4)) = v4;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> the tensor core's reads
        }
      }
      if (!ok) break;
      l += ((sum8[0] + sum8[1]) + (sum8[2] + sum8[3])) + ((sum8[4] + sum8[5]) + (sum8[6] + sum8[7]));
      if (AT_P_TMEM) tc_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) tc_mbar_arrive(&p_full[b]);
    }
    if (ok && ntiles > 0 && wait_all(&pv_done[(ntiles - 1) % AT_NBUF], ((ntiles - 1) / AT_NBUF) & 1)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const int tk = valid ? row / G : 0, h = valid ? row - tk * G : 0;
      bf16* dst = P.out + (size_t)(tok0 + tk) * P.out_stride + (size_t)(g * G + h) * HEAD_DIM;
#pragma unroll 1
      for (int cc = 0; cc < HEAD_DIM; cc += 32) {
        uint32_t ov[32];
        tc_ld32(lane_addr + AT_O_COL + cc, ov);
        if (valid) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 v4;
            v4.x = at_pack(__uint_as_float(ov[j]) * inv, __uint_as_float(ov[j + 1]) * inv);
            v4.y = at_pack(__uint_as_float(ov[j + 2]) * inv, __uint_as_float(ov[j + 3]) * inv);
            v4.z = at_pack(__uint_as_float(ov[j + 4]) * inv, __uint_as_float(ov[j + 5]) * inv);
            v4.w = at_pack(__uint_as_float(ov[j + 6]) * inv, __uint_as_float(ov[j + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + cc + j) = v4;
          }
        }
      }
    }
  }
  // ---------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(AT_TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag) report_error(P.err, PHOTON_DEV_WAIT_TIMEOUT, blockIdx.x, blockIdx.y, 0);
}

PHOTON_API int photon_attention_tc_head_dim() { return HEAD_DIM; }

// Runs the requests of the step that bring more than 16 rows (tokens x group); the others are left
// untouched.  q [T, n_q * d] with row stride q_stride, out [T, n_q * d]; k_cache, v_cache
// [num_pages, n_kv, page_size, d] contiguous.  group at most 128, page_size a multiple of 8 that
// divides 64 or is a multiple of 64.
PHOTON_API int photon_attention_tc(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                                   const void* v_cache, const int* block_table, int max_pages, const int* cu_tokens,
                                   const int* positions, int S, int max_tokens_per_seq, int T, int n_q, int n_kv, int d,
                                   int page_size, int num_pages, int window, float scale, int* err,
                                   cudaStream_t stream) {
  if (S <= 0 || T <= 0) return 0;
  if (d != HEAD_DIM || n_kv <= 0 || n_q % n_kv || !(scale > 0.f)) return PHOTON_ERR_UNSUPPORTED;
  const int G = n_q / n_kv;
  if (G > AT_ROWS) return PHOTON_ERR_UNSUPPORTED;
  if (page_size < 8 || (page_size & 7) || !((AT_KT % page_size) == 0 || (page_size % AT_KT) == 0)) return PHOTON_ERR_UNSUPPORTED;
  if (((uintptr_t)q & 15) || (q_stride & 7) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) ||
      ((uintptr_t)out & 15) || (out_stride & 7))
    return PHOTON_ERR_ARGUMENT;
  const long total_rows = (long)num_pages * n_kv * page_size;
  if (total_rows > 0x7fffffffL || n_kv > 65535) return PHOTON_ERR_UNSUPPORTED;
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return PHOTON_ERR_UNSUPPORTED;
  const int box_rows = page_size < AT_KT ? page_size : AT_KT;
  CUtensorMap map_q, map_k, map_v;
  {
    cuuint64_t dims[3] = {(cuuint64_t)d, (cuuint64_t)n_q, (cuuint64_t)T};
    cuuint64_t strides[2] = {(cuuint64_t)d * 2, (cuuint64_t)q_stride * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(AT_ROWS / G)};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return PHOTON_ERR_ARGUMENT;
  }
  int st = make_map(&map_k, k_cache, total_rows, d, d, box_rows);
  if (st != 0) return st;
  st = make_map(&map_v, v_cache, total_rows, d, d, box_rows);
  if (st != 0) return st;
  AttnTcParams P;
  P.out = (bf16*)out; P.out_stride = out_stride; P.block_table = block_table; P.max_pages = max_pages;
  P.cu_tokens = cu_tokens; P.positions = positions; P.n_kv = n_kv; P.group = G; P.tile_rows = (AT_ROWS / G) * G;
  P.page_size = page_size;
  P.num_pages = num_pages; P.box_rows = box_rows; P.window = window; P.total_rows = (int)total_rows;
  P.scale_log2 = scale * 1.4426950408889634f; P.err = err;
  const long rows = (long)max_tokens_per_seq * G;
  P.tiles_per_seq = (int)((rows + P.tile_rows - 1) / P.tile_rows);
  if ((long)S * P.tiles_per_seq > 65535) return PHOTON_ERR_UNSUPPORTED;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e1 = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM_BYTES);
    cudaError_t e2 = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e1 != cudaSuccess) return (int)e1;
    if (e2 != cudaSuccess) return (int)e2;
    attr_done = true;
  }
  dim3 grid(n_kv, S * P.tiles_per_seq);
  return launch_pdl(attention_tc_kernel, grid, dim3(AT_THREADS), (size_t)AT_SMEM_BYTES, stream, map_q, map_k, map_v, P);
}
