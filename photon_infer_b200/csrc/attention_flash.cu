// Paged causal attention on the tensor cores, for bfloat16 and head sizes that are a
// multiple of 16 up to 128: prompt portions and decoded tokens alike.
//
// The query rows of one request that share a key/value head are packed into one matrix:
// row = token_in_step * GROUP + head_in_group, so the GROUP heads that read the same keys
// read them once.  Keys and values stream from the paged cache into shared memory in
// tiles of 64 keys through a ring of cp.async stages (the block table is followed per
// key row, 16 bytes per copy); scores and the weighted sum run as mma.m16n8k16 with
// 32-bit accumulation, the softmax is a running one in 32-bit.
//
// Two shapes of work, chosen per request by its number of rows:
//   ROWS  many rows (prompt portions): a block owns 64 rows, each warp 16 of them, all
//         warps walk the same key tiles; keys after a row's own position are masked.
//   KEYS  at most 16 rows (decoded tokens): a block owns all rows, every warp takes a
//         quarter of each key tile, the keys of the request may be split over several
//         blocks; partial results are merged in a fixed order (shared memory inside a
//         block, a scratch buffer and a ticket between blocks).
//
// Formula: include/photon/ops/kernels/mha_kernel.hpp:188-229 (scores (q.k)/sqrt(d) for the
// keys up to the token's own position, softmax exp(s-max)/sum, weighted sum of values;
// head h uses key/value head h / (n_q/n_kv)), with an optional window.  The reference has
// no tensor-core kernel and no causal mask inside a portion (src/ops/kernels/cuda/
// paged_attention.cu:90-194, src/arch/transformer_block.cpp:486-509).
//
// Compiled per model with -DHEAD_DIM=<d>.
#include "common.cuh"
#include <math.h>

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif

#define FA_TILE_K 64                      // keys per tile
#ifndef FA_ROWS
#define FA_ROWS 128                       // rows per block in ROWS mode (16 per warp)
#endif
#define FA_KEYS_THREADS 128               // KEYS mode: four warps, 16 keys of every tile each
#define FA_ROWS_THREADS (FA_ROWS * 2)
#ifndef FA_STAGES
#define FA_STAGES 3
#endif
#define FA_TABLE_SMEM 256                 // block-table entries the KEYS kernel copies to shared memory up front
#define FA_LD (HEAD_DIM + 8)              // padded row length in shared memory (elements): conflict-free ldmatrix
#define FA_KD (HEAD_DIM / 16)             // k-steps over the head dimension
#define FA_ND (HEAD_DIM / 8)              // n-tiles over the head dimension

static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 128, "head size");

__device__ __forceinline__ uint32_t fa_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;           // 0: the 16 bytes are filled with zeros, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(fa_smem(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(fa_smem(p)));
}
__device__ __forceinline__ void ldsm4t(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(fa_smem(p)));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {       // 2^x; -inf gives 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct FlashParams {
  const bf16* q; long q_stride;           // [T, n_q * d] view
  bf16* out; long out_stride;             // [T, n_q * d]
  const bf16* k_cache; const bf16* v_cache;   // [pages, n_kv, page_size, d]
  const int* block_table; int max_pages;  // [S, max_pages]
  const int* cu_tokens;                   // [S + 1] first token of each request in the step
  const int* positions;                   // [T]
  const int* context_lens;                // [S] or null: tokens of the request after this step; when given, the
                                          // KEYS kernel takes a request's positions as context_len - n .. context_len - 1
  float* part_acc; float* part_ml; int* tickets;   // scratch of the KEYS mode with splits
  int n_q, n_kv, group, page_size, page_shift, num_pages, window, num_splits, tiles_per_seq;   // page_shift: log2(page_size) or -1
  float scale_log2;                       // scale * log2(e)
  int* err;
};

// Copies the keys [key0, key0 + 64) of key/value head g into one stage (K tile, then V tile).
// Rows outside [lo, hi] or without a page are filled with zeros.
// tid, nthreads: the calling thread's index in the group of threads that share this stage, and the group's size.
__device__ __forceinline__ void load_kv_tile(const FlashParams& P, const int* table, const int* table_s, int g,
                                             int key0, int lo, int hi, bf16* ks, bf16* vs, int t_for_err,
                                             int tid, int nthreads) {
  constexpr int CPR = HEAD_DIM / 8;                       // 16-byte chunks per row
  for (int c = tid; c < FA_TILE_K * CPR; c += nthreads) {
    const int r = c / CPR, cc = c - r * CPR;
    const int key = key0 + r;
    bool valid = key >= lo && key <= hi;
    size_t src = 0;
    if (valid) {
      const int pidx = P.page_shift >= 0 ? (key >> P.page_shift) : key / P.page_size;
      const int slot = P.page_shift >= 0 ? (key & (P.page_size - 1)) : key - pidx * P.page_size;
      const int page = (table_s != nullptr && pidx < FA_TABLE_SMEM) ? table_s[pidx] : table[pidx];
      if (page < 0 || page >= P.num_pages) {
        if (cc == 0) report_error(P.err, PHOTON_DEV_BAD_PAGE, t_for_err, key, page);
        valid = false;
      } else {
        src = (((size_t)page * P.n_kv + g) * P.page_size + slot) * HEAD_DIM + cc * 8;
      }
    }
    cp_async16(ks + r * FA_LD + cc * 8, P.k_cache + src, valid);
    cp_async16(vs + r * FA_LD + cc * 8, P.v_cache + src, valid);
  }
}

// One warp: scores of its 16 rows against NT*8 keys starting at key row `krow` of the K tile, running
// softmax, weighted sum with the same keys of the V tile.  qa: the rows' A fragments.  pos0/pos1 and
// lo0/lo1: last and first visible key of the lane's two rows (row lane/4 and lane/4 + 8).
// MASK false: every key of the tile is visible to every row of the warp (the caller has checked), so
// the comparisons are left out.
template <int NT, bool MASK>
__device__ __forceinline__ void warp_tile(const uint32_t (&qa)[FA_KD][4], const bf16* ks, const bf16* vs, int krow,
                                          int key_base, int pos0, int pos1, int lo0, int lo1, float scale_log2,
                                          float (&m)[2], float (&l)[2], float (&o)[FA_ND][4]) {
  const int lane = threadIdx.x & 31;
  float s[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
  // S = Q K^T
#pragma unroll
  for (int kd = 0; kd < FA_KD; ++kd) {
#pragma unroll
    for (int j = 0; j < NT; j += 2) {
      uint32_t b[4];
      const int key = krow + j * 8 + (lane & 7) + ((lane >> 4) << 3);
      const int dim = kd * 16 + (((lane >> 3) & 1) << 3);
      ldsm4(b, ks + key * FA_LD + dim);
      mma_bf16(s[j], qa[kd], b[0], b[1]);
      mma_bf16(s[j + 1], qa[kd], b[2], b[3]);
    }
  }
  // scale, mask, running softmax (base 2); the scale is applied inside the exponent: 2^(s*c - m*c)
  const int c2 = (lane & 3) * 2;
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    if (MASK) {
      const int key = key_base + krow + j * 8 + c2;
      s[j][0] = (key >= lo0 && key <= pos0) ? s[j][0] : -INFINITY;
      s[j][1] = (key + 1 >= lo0 && key + 1 <= pos0) ? s[j][1] : -INFINITY;
      s[j][2] = (key >= lo1 && key <= pos1) ? s[j][2] : -INFINITY;
      s[j][3] = (key + 1 >= lo1 && key + 1 <= pos1) ? s[j][3] : -INFINITY;
    }
    mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
    mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  // m holds the running maximum of the scaled scores (scale_log2 > 0, so the order is kept)
  const float mn0 = fmaxf(m[0], mx0 * scale_log2), mn1 = fmaxf(m[1], mx1 * scale_log2);
  const float sub0 = (mn0 == -INFINITY) ? 0.f : mn0, sub1 = (mn1 == -INFINITY) ? 0.f : mn1;
  const float corr0 = fast_exp2(m[0] - sub0);             // 2^(-inf) = 0 for the first tile
  const float corr1 = fast_exp2(m[1] - sub1);
  m[0] = mn0; m[1] = mn1;
  float sum0 = 0.f, sum1 = 0.f;
  uint32_t pa[NT / 2][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const float p0 = fast_exp2(fmaf(s[j][0], scale_log2, -sub0)), p1 = fast_exp2(fmaf(s[j][1], scale_log2, -sub0));
    const float p2 = fast_exp2(fmaf(s[j][2], scale_log2, -sub1)), p3 = fast_exp2(fmaf(s[j][3], scale_log2, -sub1));
    sum0 += p0 + p1; sum1 += p2 + p3;
    pa[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);
    pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
  }
  l[0] = l[0] * corr0 + sum0;             // per-lane partial sums; the quad is added up at the end
  l[1] = l[1] * corr1 + sum1;
#pragma unroll
  for (int n = 0; n < FA_ND; ++n) { o[n][0] *= corr0; o[n][1] *= corr0; o[n][2] *= corr1; o[n][3] *= corr1; }
  // O += P V
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
#pragma unroll
    for (int n = 0; n < FA_ND; n += 2) {
      uint32_t b[4];
      const int key = krow + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const int dim = n * 8 + ((lane >> 4) << 3);
      ldsm4t(b, vs + key * FA_LD + dim);
      mma_bf16(o[n], pa[kk], b[0], b[1]);
      mma_bf16(o[n + 1], pa[kk], b[2], b[3]);
    }
  }
}

// NSUB (KEYS mode): groups of four warps in a block; each group walks its own share of the block's key
// tiles with a ring of stages of its own, and the groups' results are merged through shared memory like
// the warps' (one block per SM then does what NSUB blocks with a merge through global memory would).
// STAGES: depth of a group's ring of key/value tiles.  Three keep a block's loads two tiles ahead; two make
// room for five blocks per SM instead of three, which pays when there are more blocks than places.
template <bool KEYS_MODE, int NSUB, int STAGES>
__global__ void __launch_bounds__(KEYS_MODE ? FA_KEYS_THREADS * NSUB : FA_ROWS_THREADS,
                                  KEYS_MODE ? (NSUB == 1 ? (STAGES == 2 ? 4 : 3) : 1) : (FA_ROWS >= 128 ? 2 : 3))
flash_attention_kernel(const FlashParams P) {
  extern __shared__ __align__(16) unsigned char fa_dyn[];
  constexpr int Q_ELEMS = (KEYS_MODE ? 16 : FA_ROWS) * FA_LD;
  constexpr int RING_ELEMS = STAGES * 2 * FA_TILE_K * FA_LD;
  const int sub = KEYS_MODE ? (int)(threadIdx.x >> 7) : 0;                  // group of four warps
  const int stid = KEYS_MODE ? (int)(threadIdx.x & 127) : (int)threadIdx.x; // thread index inside the group
  const int sthreads = KEYS_MODE ? FA_KEYS_THREADS : FA_ROWS_THREADS;
  // per group: Q rows (KEYS: 16, ROWS: FA_ROWS) x FA_LD, then STAGES x (K | V) x 64 x FA_LD
  bf16* qs = reinterpret_cast<bf16*>(fa_dyn) + (size_t)sub * (Q_ELEMS + RING_ELEMS);
  bf16* kv = qs + Q_ELEMS;
  auto group_sync = [&]() {
    if (KEYS_MODE && NSUB > 1) asm volatile("bar.sync %0, 128;" ::"r"(sub + 1) : "memory");
    else __syncthreads();
  };
  __shared__ int s_flag;

  __shared__ int table_s[KEYS_MODE ? FA_TABLE_SMEM : 1];
  pdl_wait();
  const int split = blockIdx.x, g = blockIdx.y;
  // row tiles are handed out last-first: the tiles with the most keys to walk start first
  const int seq = blockIdx.z / P.tiles_per_seq, qtile = P.tiles_per_seq - 1 - (blockIdx.z - seq * P.tiles_per_seq);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wq = warp & 3;                                                  // KEYS: the warp's quarter of a key tile
  const int G = P.group;
  const int* table = P.block_table + (size_t)seq * P.max_pages;
  if (KEYS_MODE) {
    // The request's block-table row goes to shared memory in the same round trip as its token range and
    // length: the key loads then depend on one memory latency, not on three in a row.
    for (int i = threadIdx.x; i < min(P.max_pages, FA_TABLE_SMEM); i += blockDim.x) table_s[i] = table[i];
  }
  const int tok0 = P.cu_tokens[seq], tok1 = P.cu_tokens[seq + 1];
  const int ctx_len = (KEYS_MODE && P.context_lens != nullptr) ? P.context_lens[seq] : -1;
  const int ntok = tok1 - tok0;
  const int rows = ntok * G;
  if ((rows <= 16) != KEYS_MODE) return;                                   // the other launch takes this request
  const int row0 = KEYS_MODE ? 0 : qtile * FA_ROWS;
  if (row0 >= rows || (KEYS_MODE && qtile > 0)) return;
  const int nrows = min(KEYS_MODE ? 16 : FA_ROWS, rows - row0);
  const bool by_len = KEYS_MODE && ctx_len >= 0;                           // positions follow from the length

  // positions of the tile's first and last token bound the keys the block needs
  const int tfirst = row0 / G, tlast = (row0 + nrows - 1) / G;
  const int pos_first = by_len ? ctx_len - ntok + tfirst : P.positions[tok0 + tfirst];
  const int pos_last = by_len ? ctx_len - ntok + tlast : P.positions[tok0 + tlast];
  const int key_lo = (P.window > 0 && pos_first - P.window + 1 > 0) ? pos_first - P.window + 1 : 0;
  int tile_begin = key_lo / FA_TILE_K, tile_end = pos_last / FA_TILE_K + 1;     // key tiles [begin, end)
  if (KEYS_MODE && P.num_splits > 1) {
    const int per = (tile_end - tile_begin + P.num_splits - 1) / P.num_splits;
    tile_begin += split * per;
    tile_end = min(tile_end, tile_begin + per);
  }
  if (KEYS_MODE && NSUB > 1) {
    // the block's tiles are dealt to its groups in order
    const int per = (max(0, tile_end - tile_begin) + NSUB - 1) / NSUB;
    tile_begin += sub * per;
    tile_end = min(tile_end, tile_begin + per);
  }
  const int ntiles = max(0, tile_end - tile_begin);
  if (KEYS_MODE) __syncthreads();                                          // table_s is complete
  const int* tsm = KEYS_MODE ? table_s : nullptr;

  // ---- Q rows into shared memory (zeros beyond the valid rows)
  {
    constexpr int CPR = HEAD_DIM / 8;
    const int qrows = KEYS_MODE ? 16 : FA_ROWS;
    for (int c = stid; c < qrows * CPR; c += sthreads) {                   // KEYS: every group has a copy of its own
      const int r = c / CPR, cc = c - r * CPR;
      const int row = row0 + r;
      const bool valid = row < rows;
      const int tk = valid ? row / G : 0, h = valid ? row - tk * G : 0;
      cp_async16(qs + r * FA_LD + cc * 8,
                 P.q + (size_t)(tok0 + tk) * P.q_stride + (size_t)(g * G + h) * HEAD_DIM + cc * 8, valid);
    }
  }
  auto stage_k = [&](int st) { return kv + (size_t)st * 2 * FA_TILE_K * FA_LD; };
  auto stage_v = [&](int st) { return kv + (size_t)st * 2 * FA_TILE_K * FA_LD + FA_TILE_K * FA_LD; };
  // prologue: the first STAGES - 1 tiles (the Q copy joins the first group)
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {
    if (i < ntiles) load_kv_tile(P, table, tsm, g, (tile_begin + i) * FA_TILE_K, key_lo, pos_last, stage_k(i), stage_v(i), tok0, stid, sthreads);
    cp_async_commit();
  }

  // ---- per-lane row data
  const int wrow = KEYS_MODE ? 0 : warp * 16;                              // first row of the warp inside the tile
  int pos_r[2], lo_r[2];
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    const int row = row0 + wrow + (lane >> 2) + h2 * 8;
    if (row < rows) {
      pos_r[h2] = by_len ? ctx_len - ntok + row / G : P.positions[tok0 + row / G];
      lo_r[h2] = (P.window > 0 && pos_r[h2] - P.window + 1 > 0) ? pos_r[h2] - P.window + 1 : 0;
    } else {
      pos_r[h2] = -1; lo_r[h2] = 0;                                        // sees nothing
    }
  }
  int warp_pos_max = max(pos_r[0], pos_r[1]);
  int warp_pos_min = min(pos_r[0], pos_r[1]);             // -1 when the warp has a row beyond the request's rows
  int warp_lo_max = max(lo_r[0], lo_r[1]);
#pragma unroll
  for (int o2 = 16; o2 > 0; o2 >>= 1) {
    warp_pos_max = max(warp_pos_max, __shfl_xor_sync(0xffffffffu, warp_pos_max, o2));
    warp_pos_min = min(warp_pos_min, __shfl_xor_sync(0xffffffffu, warp_pos_min, o2));
    warp_lo_max = max(warp_lo_max, __shfl_xor_sync(0xffffffffu, warp_lo_max, o2));
  }

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[FA_ND][4];
#pragma unroll
  for (int n = 0; n < FA_ND; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  uint32_t qa[FA_KD][4];

  for (int i = 0; i < ntiles; ++i) {
    // keep STAGES - 1 tiles in flight
    {
      const int nx = i + STAGES - 1;
      if (nx < ntiles)
        load_kv_tile(P, table, tsm, g, (tile_begin + nx) * FA_TILE_K, key_lo, pos_last, stage_k(nx % STAGES),
                     stage_v(nx % STAGES), tok0, stid, sthreads);
      cp_async_commit();
    }
    cp_async_wait<STAGES - 1>();
    group_sync();
    if (i == 0) {
#pragma unroll
      for (int kd = 0; kd < FA_KD; ++kd)
        ldsm4(qa[kd], qs + (wrow + (lane & 15)) * FA_LD + kd * 16 + ((lane >> 4) << 3));
    }
    const int st = i % STAGES;
    const int key_base = (tile_begin + i) * FA_TILE_K;
    if (KEYS_MODE) {
      // every warp takes 16 keys of the tile
      const int k0 = key_base + wq * 16;
      if (k0 <= warp_pos_max) {
        if (k0 + 15 <= warp_pos_min && k0 >= warp_lo_max)
          warp_tile<2, false>(qa, stage_k(st), stage_v(st), wq * 16, key_base, pos_r[0], pos_r[1], lo_r[0], lo_r[1],
                              P.scale_log2, m, l, o);
        else
          warp_tile<2, true>(qa, stage_k(st), stage_v(st), wq * 16, key_base, pos_r[0], pos_r[1], lo_r[0], lo_r[1],
                             P.scale_log2, m, l, o);
      }
    } else {
      if (key_base <= warp_pos_max) {                                      // tiles after the warp's last row are skipped
        if (key_base + FA_TILE_K - 1 <= warp_pos_min && key_base >= warp_lo_max)
          warp_tile<8, false>(qa, stage_k(st), stage_v(st), 0, key_base, pos_r[0], pos_r[1], lo_r[0], lo_r[1],
                              P.scale_log2, m, l, o);
        else
          warp_tile<8, true>(qa, stage_k(st), stage_v(st), 0, key_base, pos_r[0], pos_r[1], lo_r[0], lo_r[1],
                             P.scale_log2, m, l, o);
      }
    }
    group_sync();                                                          // the stage may be overwritten
  }
  cp_async_wait<0>();
  pdl_launch_dependents();                         // the next kernel may be scheduled while the results are merged

  // the quad's partial sums
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    l[h2] += __shfl_xor_sync(0xffffffffu, l[h2], 1);
    l[h2] += __shfl_xor_sync(0xffffffffu, l[h2], 2);
  }

  if (!KEYS_MODE) {
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      const int row = row0 + wrow + (lane >> 2) + h2 * 8;
      if (row >= rows) continue;
      const int tk = row / G, h = row - tk * G;
      const float inv = l[h2] > 0.f ? 1.f / l[h2] : 0.f;
      bf16* dst = P.out + (size_t)(tok0 + tk) * P.out_stride + (size_t)(g * G + h) * HEAD_DIM + (lane & 3) * 2;
#pragma unroll
      for (int n = 0; n < FA_ND; ++n)
        *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = __floats2bfloat162_rn(o[n][h2 * 2] * inv, o[n][h2 * 2 + 1] * inv);
    }
    return;
  }

  // ---- KEYS mode: merge the warps (each saw its own keys) through shared memory, in warp order
  constexpr int NW = 4 * NSUB;
  __syncthreads();                                                         // all warps are done with the rings
  float* wm = reinterpret_cast<float*>(fa_dyn);                            // [NW][16]
  float* wl = wm + NW * 16;                                                // [NW][16]
  float* wo = wl + NW * 16;                                                // [NW][16][HEAD_DIM]
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    const int r = (lane >> 2) + h2 * 8;
    if ((lane & 3) == 0) { wm[warp * 16 + r] = m[h2]; wl[warp * 16 + r] = l[h2]; }
#pragma unroll
    for (int n = 0; n < FA_ND; ++n) {
      wo[(warp * 16 + r) * HEAD_DIM + n * 8 + (lane & 3) * 2] = o[n][h2 * 2];
      wo[(warp * 16 + r) * HEAD_DIM + n * 8 + (lane & 3) * 2 + 1] = o[n][h2 * 2 + 1];
    }
  }
  __syncthreads();
  const int n_q = P.n_kv * G;
  for (int e = threadIdx.x; e < nrows * HEAD_DIM; e += blockDim.x) {
    const int r = e / HEAD_DIM, d = e - r * HEAD_DIM;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, wm[w * 16 + r]);
    float L = 0.f, A = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float mw = wm[w * 16 + r];
        const float sc = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        L += wl[w * 16 + r] * sc;
        A += wo[(w * 16 + r) * HEAD_DIM + d] * sc;
      }
    }
    const int tk = r / G, h = r - tk * G;
    const int head = g * G + h;
    if (P.num_splits == 1) {
      P.out[(size_t)(tok0 + tk) * P.out_stride + (size_t)head * HEAD_DIM + d] = __float2bfloat16_rn(L > 0.f ? A / L : 0.f);
    } else {
      const size_t slot = ((size_t)(tok0 + tk) * n_q + head) * P.num_splits + split;
      __stcg(P.part_acc + slot * HEAD_DIM + d, A);
      if (d == 0) { __stcg(P.part_ml + slot * 2, M); __stcg(P.part_ml + slot * 2 + 1, L); }
    }
  }
  if (P.num_splits == 1) return;
  // the block that draws the last ticket of (request, key/value head) merges the shares in split order
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_flag = (atomicAdd(P.tickets + (size_t)seq * P.n_kv + g, 1) == P.num_splits - 1);
  __syncthreads();
  if (!s_flag) return;
  __threadfence();
  if (threadIdx.x == 0) P.tickets[(size_t)seq * P.n_kv + g] = 0;
  for (int e = threadIdx.x; e < nrows * HEAD_DIM; e += blockDim.x) {
    const int r = e / HEAD_DIM, d = e - r * HEAD_DIM;
    const int tk = r / G, h = r - tk * G;
    const int head = g * G + h;
    const size_t base = ((size_t)(tok0 + tk) * n_q + head) * P.num_splits;
    float M = -INFINITY;
    for (int s2 = 0; s2 < P.num_splits; ++s2) M = fmaxf(M, __ldcg(P.part_ml + (base + s2) * 2));
    float L = 0.f, A = 0.f;
    if (M != -INFINITY) {
      for (int s2 = 0; s2 < P.num_splits; ++s2) {
        const float ms = __ldcg(P.part_ml + (base + s2) * 2);
        const float sc = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
        L += __ldcg(P.part_ml + (base + s2) * 2 + 1) * sc;
        A += __ldcg(P.part_acc + (base + s2) * HEAD_DIM + d) * sc;
      }
    }
    P.out[(size_t)(tok0 + tk) * P.out_stride + (size_t)head * HEAD_DIM + d] = __float2bfloat16_rn(L > 0.f ? A / L : 0.f);
  }
}

PHOTON_API int photon_flash_attention_head_dim() { return HEAD_DIM; }
// Groups of four warps (each with a ring of stages of its own) that fit into the shared memory of one block.
constexpr int FA_GROUP_BYTES = (16 * FA_LD + FA_STAGES * 2 * FA_TILE_K * FA_LD) * 2;
constexpr int FA_MAX_GROUPS = (4 * FA_GROUP_BYTES + 2048 <= 232448) ? 4 : ((2 * FA_GROUP_BYTES + 2048 <= 232448) ? 2 : 1);
PHOTON_API int photon_flash_attention_max_groups() { return FA_MAX_GROUPS; }

// mode bit 0: launch the ROWS kernel (requests with more than 16 rows); bit 1: the KEYS kernel (at most 16
// rows = tokens * group).  max_tokens_per_seq bounds the tokens any request brings in this step.
// nsub: 1, 2 or 4 groups of four warps per block of the KEYS kernel, each walking its own share of the block's
// key tiles (at most photon_flash_attention_max_groups(), which depends on the head size).
// context_lens (may be null): tokens of each request after this step; with it the KEYS kernel does not read
// `positions` (the tokens a request brings are then taken to be its last ones, in order).
// Scratch (KEYS mode with num_splits > 1): part_acc float [T * n_q * num_splits * d], part_ml float
// [T * n_q * num_splits * 2], tickets int [S * n_kv] all zero between launches.  Launches that share scratch
// must not overlap on the device.
PHOTON_API int photon_flash_attention(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                                      const void* v_cache, const int* block_table, int max_pages,
                                      const int* cu_tokens, const int* positions, const int* context_lens,
                                      float* part_acc, float* part_ml,
                                      int* tickets, int S, int max_tokens_per_seq, int n_q, int n_kv, int d,
                                      int page_size, int num_pages, int window, float scale, int num_splits,
                                      int nsub, int mode, int* err, cudaStream_t stream) {
  if (S <= 0) return 0;
  if (d != HEAD_DIM || n_kv <= 0 || n_q % n_kv || !(scale > 0.f)) return PHOTON_ERR_UNSUPPORTED;
  if (((uintptr_t)q % 16) || ((size_t)q_stride * 2) % 16 || ((uintptr_t)k_cache % 16) || ((uintptr_t)v_cache % 16))
    return PHOTON_ERR_ARGUMENT;
  if (num_splits < 1 || num_splits > 65535 || n_kv > 65535) return PHOTON_ERR_UNSUPPORTED;
  if (num_splits > 1 && (part_acc == nullptr || part_ml == nullptr || tickets == nullptr)) return PHOTON_ERR_ARGUMENT;
  FlashParams P;
  P.q = (const bf16*)q; P.q_stride = q_stride; P.out = (bf16*)out; P.out_stride = out_stride;
  P.k_cache = (const bf16*)k_cache; P.v_cache = (const bf16*)v_cache;
  P.block_table = block_table; P.max_pages = max_pages; P.cu_tokens = cu_tokens; P.positions = positions;
  P.context_lens = context_lens;
  P.part_acc = part_acc; P.part_ml = part_ml; P.tickets = tickets;
  P.n_q = n_q; P.n_kv = n_kv; P.group = n_q / n_kv; P.page_size = page_size; P.num_pages = num_pages;
  P.page_shift = -1;
  for (int sh = 0; sh < 20; ++sh) if ((1 << sh) == page_size) P.page_shift = sh;
  P.window = window; P.scale_log2 = scale * 1.4426950408889634f; P.err = err;
  const size_t ring = (size_t)FA_STAGES * 2 * FA_TILE_K * FA_LD;
  const size_t ring2 = (size_t)2 * 2 * FA_TILE_K * FA_LD;                   // two stages
  const size_t smem_rows = ((size_t)FA_ROWS * FA_LD + ring) * sizeof(bf16);
  const size_t smem_keys = ((size_t)16 * FA_LD + ring) * sizeof(bf16);      // per group of four warps
  const size_t smem_keys2 = ((size_t)16 * FA_LD + ring2) * sizeof(bf16);
  if (nsub != 1 && nsub != 2 && nsub != 4) return PHOTON_ERR_ARGUMENT;
  if (nsub > photon_flash_attention_max_groups()) return PHOTON_ERR_UNSUPPORTED;
  static bool attr_done = false;
  if (!attr_done) {
    // room for several blocks per SM: the largest shared-memory carve-out
    cudaError_t e[10];
    e[0] = cudaFuncSetAttribute(flash_attention_kernel<false, 1, FA_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_rows);
    e[1] = cudaFuncSetAttribute(flash_attention_kernel<false, 1, FA_STAGES>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    e[2] = cudaFuncSetAttribute(flash_attention_kernel<true, 1, FA_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_keys);
    e[3] = cudaFuncSetAttribute(flash_attention_kernel<true, 1, FA_STAGES>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    e[8] = cudaFuncSetAttribute(flash_attention_kernel<true, 1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_keys2);
    e[9] = cudaFuncSetAttribute(flash_attention_kernel<true, 1, 2>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    e[4] = e[5] = e[6] = e[7] = cudaSuccess;
    if (photon_flash_attention_max_groups() >= 2) {
      e[4] = cudaFuncSetAttribute(flash_attention_kernel<true, 2, FA_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * smem_keys));
      e[5] = cudaFuncSetAttribute(flash_attention_kernel<true, 2, FA_STAGES>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    }
    if (photon_flash_attention_max_groups() >= 4) {
      e[6] = cudaFuncSetAttribute(flash_attention_kernel<true, 4, FA_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(4 * smem_keys));
      e[7] = cudaFuncSetAttribute(flash_attention_kernel<true, 4, FA_STAGES>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    }
    for (int i = 0; i < 10; ++i) if (e[i] != cudaSuccess) return (int)e[i];
    attr_done = true;
  }
  if (mode & 1) {
    const int rows = max_tokens_per_seq * P.group;
    P.tiles_per_seq = (rows + FA_ROWS - 1) / FA_ROWS;
    P.num_splits = 1;
    if ((long)S * P.tiles_per_seq > 65535) return PHOTON_ERR_UNSUPPORTED;
    dim3 grid(1, n_kv, S * P.tiles_per_seq);
    int st = launch_pdl(flash_attention_kernel<false, 1, FA_STAGES>, grid, dim3(FA_ROWS_THREADS), smem_rows, stream, P);
    if (st != 0) return st;
  }
  if (mode & 2) {
    P.tiles_per_seq = 1;
    P.num_splits = num_splits;
    if (S > 65535) return PHOTON_ERR_UNSUPPORTED;
    dim3 grid(num_splits, n_kv, S);
    if (nsub == 4) {
      if constexpr (FA_MAX_GROUPS >= 4)
        return launch_pdl(flash_attention_kernel<true, 4, FA_STAGES>, grid, dim3(FA_KEYS_THREADS * 4), 4 * smem_keys, stream, P);
    } else if (nsub == 2) {
      if constexpr (FA_MAX_GROUPS >= 2)
        return launch_pdl(flash_attention_kernel<true, 2, FA_STAGES>, grid, dim3(FA_KEYS_THREADS * 2), 2 * smem_keys, stream, P);
    }
    // more blocks than the places that rings of three stages leave (three per SM at heads of 64): rings of two stages
    // (measured at 32/8 heads of 64, 640 keys, batch 64: 22.0 us against 31.6 us)
    static int places3 = 0;
    if (places3 == 0) {
      int dev = 0, sms = 0;
      cudaGetDevice(&dev);
      if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
      places3 = sms * (int)(232448 / (smem_keys + 1024));                  // blocks that fit by shared memory
    }
    if ((long)num_splits * n_kv * S > places3)
      return launch_pdl(flash_attention_kernel<true, 1, 2>, grid, dim3(FA_KEYS_THREADS), smem_keys2, stream, P);
    return launch_pdl(flash_attention_kernel<true, 1, FA_STAGES>, grid, dim3(FA_KEYS_THREADS), smem_keys, stream, P);
  }
  return 0;
}
