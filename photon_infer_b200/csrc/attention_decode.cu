// Paged attention of decoded tokens for large batches and long contexts, bfloat16, head size 64 or 128.
//
// The requests of a step that bring at most 16 query rows (row = token_in_step * GROUP + head_in_group, the
// packing of attention_flash.cu) have their keys cut into chunks of tiles of 64 keys.  A work item is
// (request, key/value head, chunk).  The grid is persistent: as many blocks as the GPU holds at once, each
// drawing items from a counter, so a step whose (request, head) pairs slightly outnumber the places does not
// pay for a second, nearly empty wave, and requests of very different lengths weigh what they weigh.  The item
// list follows from the requests' lengths inside the kernel (a prefix sum over the requests), so a captured
// graph serves every step of its shape; the host gives a chunk length for the longest context the block table
// allows, and the kernel shortens or lengthens it by the same rule for what requests of nearly one length
// hold now.
//
// Keys and values come by TMA: one 2-D box per page part (16 keys x 64 features with pages of 16), 128-byte
// swizzle, into a ring of stages, completion on an mbarrier.  Four producer warps (they give their registers
// to the others with setmaxnreg) issue a page part each, because a TMA instruction costs its thread 150 to 200
// cycles and a tile is eight or sixteen of them; one of them draws the items and hands them to the consumers
// through a small queue.  (The 2,048 cp.async instructions with their address arithmetic that a tile costs in
// attention_flash.cu made that kernel issue-bound: 47 % of all issue slots at 18 % occupancy.)  The four
// consumer warps take 16 keys of every tile each: scores and weighted sums as mma.m16n8k16 with fragments read
// by ldmatrix from the swizzled tiles, running softmax in 32-bit, merged in warp order through shared memory.
// A request with one chunk is written out directly; otherwise the item leaves (max, sum, weighted sum) in a
// scratch buffer and the block that draws the last ticket of (request, head) merges the chunks in chunk order.
//
// Keys beyond a row's position are masked by selection, so stale key rows do not matter; value rows outside
// the visible range are set to zero in shared memory before the product reads them (P = 0 times a stale
// NaN would still be NaN).  Page parts wholly outside the range are not read (TMA zero fill).
//
// Formula: include/photon/ops/kernels/mha_kernel.hpp:188-229; the reference's paged kernel walks every key
// with one thread and adds 1e-6 to the softmax sum (src/ops/kernels/cuda/paged_attention.cu:71,132-160),
// neither of which is reproduced.
//
// Compiled per model with -DHEAD_DIM=<64|128>.  Every mbarrier wait is bounded (PHOTON_DEV_WAIT_TIMEOUT).
#include "tcgen05.cuh"
#include <math.h>

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
static_assert(HEAD_DIM == 64 || HEAD_DIM == 128, "head size of the TMA decode attention");

#define AD_TILE 64                                  // keys per tile
#define AD_THREADS 256                              // warps 0-3: the keys, warps 4-7: TMA
#define AD_DH (HEAD_DIM / 64)                       // 64-wide halves of the head dimension
#define AD_HALF_BYTES (AD_TILE * 128)               // one 64-wide half of a K or V tile
#define AD_KV_BYTES (AD_TILE * HEAD_DIM * 2)        // one K tile or one V tile
#define AD_STAGE_BYTES (2 * AD_KV_BYTES)
#ifndef AD_STAGES
#define AD_STAGES (HEAD_DIM == 64 ? 5 : 3)           // two blocks per SM either way
#endif
#define AD_QLD (HEAD_DIM + 8)                       // padded row of Q in shared memory (elements)
#define AD_KD (HEAD_DIM / 16)
#define AD_ND (HEAD_DIM / 8)
#define AD_MAX_SEQS 512
#ifndef AD_ADAPTIVE
#define AD_ADAPTIVE 1                              // 0: the host's chunk size is used as it is (for comparisons)
#endif
#define AD_MAX_CHUNKS (HEAD_DIM < 120 ? HEAD_DIM : 120)   // chunks of one request: 16 rows x (chunks + 1) weights fit the merge buffer of 16 x (HEAD_DIM + 2) floats; a lane holds four
#define AD_Q_BYTES (16 * HEAD_DIM * 2)              // the 16 query rows
#define AD_MERGE_BYTES (16 * (HEAD_DIM + 2) * 4)    // one warp's partial result
#define AD_SMEM_BYTES (AD_STAGES * AD_STAGE_BYTES + AD_Q_BYTES + AD_MERGE_BYTES + 1024)

#ifdef AD_TRACE
__device__ unsigned long long ad_trace[8];        // cycles of block 0: [0] producer wait, [1] producer total, [2] consumer wait,
                                                  // [3] consumer tiles, [4] consumer merge and store, [5] consumer total, [6] tiles, [7] items
PHOTON_API int photon_attention_decode_trace(unsigned long long* host) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(host, ad_trace, sizeof(ad_trace));
  unsigned long long zero[8] = {0};
  cudaMemcpyToSymbol(ad_trace, zero, sizeof(zero));
  return 0;
}
#define AD_T(...) __VA_ARGS__
#else
#define AD_T(...)
#endif

// A work item: (request, key/value head, chunk) and its tiles.  ntiles < 0: no more items.
struct Item { int seq, g, chunk, nchunks, tok0, ntok, ctx, tile_begin, ntiles, key_lo, pos_last; };
#define AD_QUEUE 4                                  // items the producer may be ahead of the consumers

struct DecodeParams {
  const bf16* q; long q_stride;            // [T, n_q * d] view
  bf16* out; long out_stride;              // [T, n_q * d]
  const int* block_table; int max_pages;   // [S, max_pages]
  const int* cu_tokens;                    // [S + 1]
  const int* context_lens;                 // [S] tokens of each request after this step
  float* part_acc; float* part_ml; long scratch_chunks;   // room for this many (request, chunk) pairs
  int* tickets;                            // [S * n_kv] tickets, then the counter of items handed out and the counter of
                                           // blocks that are done; all zero between launches
  int S, n_kv, group, page_size, num_pages, total_rows, box_rows, window, chunk_tiles;
  int q_rows;                              // rows of the Q box: GROUP * floor(16 / GROUP)
  int T;                                   // tokens of the step (rows of q and out)
  float scale_log2;
  int* err;
};

__device__ __forceinline__ void ad_ldsm4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ad_ldsm4t(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ad_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ad_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t ad_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void ad_cp16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(tc_smem(dst)), "l"(src), "r"(n) : "memory");
}
// Byte offset of (key row, feature) inside a K or V tile: halves of 64 features, rows of 128 bytes whose
// 16-byte pieces are permuted by the row's low three bits (the TMA's 128-byte swizzle).
__device__ __forceinline__ uint32_t ad_off(int key, int dim) {
  return (uint32_t)((dim >> 6) * AD_HALF_BYTES + key * 128 + ((((dim & 63) >> 3) ^ (key & 7)) << 4));
}

// One warp: scores of the 16 query rows against 16 keys from row `krow` of the tile, running softmax, weighted
// sum with the same rows of the V tile.  MASK false: every one of the 16 keys is visible to every row.
template <bool MASK>
__device__ __forceinline__ void ad_warp_tile(const uint32_t (&qa)[AD_KD][4], uint32_t ks, uint32_t vs, int krow,
                                             int key_base, int pos0, int pos1, int lo0, int lo1, float scale_log2,
                                             float (&m)[2], float (&l)[2], float (&o)[AD_ND][4]) {
  const int lane = threadIdx.x & 31;
  float s[2][4];
#pragma unroll
  for (int j = 0; j < 2; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
  for (int kd = 0; kd < AD_KD; ++kd) {
    uint32_t b[4];
    const int key = krow + (lane & 7) + ((lane >> 4) << 3);
    const int dim = kd * 16 + (((lane >> 3) & 1) << 3);
    ad_ldsm4(b, ks + ad_off(key, dim));
    ad_mma(s[0], qa[kd], b[0], b[1]);
    ad_mma(s[1], qa[kd], b[2], b[3]);
  }
  const int c2 = (lane & 3) * 2;
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
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
  const float mn0 = fmaxf(m[0], mx0 * scale_log2), mn1 = fmaxf(m[1], mx1 * scale_log2);
  const float sub0 = (mn0 == -INFINITY) ? 0.f : mn0, sub1 = (mn1 == -INFINITY) ? 0.f : mn1;
  const float corr0 = ad_exp2(m[0] - sub0), corr1 = ad_exp2(m[1] - sub1);
  // rescale only when some row's maximum moved (uniform for the warp)
  const bool moved = __any_sync(0xffffffffu, mn0 != m[0] || mn1 != m[1]);
  m[0] = mn0; m[1] = mn1;
  float sum0 = 0.f, sum1 = 0.f;
  uint32_t pa[4];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float p0 = ad_exp2(fmaf(s[j][0], scale_log2, -sub0)), p1 = ad_exp2(fmaf(s[j][1], scale_log2, -sub0));
    const float p2 = ad_exp2(fmaf(s[j][2], scale_log2, -sub1)), p3 = ad_exp2(fmaf(s[j][3], scale_log2, -sub1));
    sum0 += p0 + p1; sum1 += p2 + p3;
    pa[j * 2] = ad_pack(p0, p1);
    pa[j * 2 + 1] = ad_pack(p2, p3);
  }
  if (moved) {
    l[0] *= corr0; l[1] *= corr1;
#pragma unroll
    for (int n = 0; n < AD_ND; ++n) { o[n][0] *= corr0; o[n][1] *= corr0; o[n][2] *= corr1; o[n][3] *= corr1; }
  }
  l[0] += sum0; l[1] += sum1;                       // per-lane partial sums; the quad is added up at the end
#pragma unroll
  for (int n = 0; n < AD_ND; n += 2) {
    uint32_t b[4];
    const int key = krow + (lane & 7) + (((lane >> 3) & 1) << 3);
    const int dim = n * 8 + ((lane >> 4) << 3);
    ad_ldsm4t(b, vs + ad_off(key, dim));
    ad_mma(o[n], pa, b[0], b[1]);
    ad_mma(o[n + 1], pa, b[2], b[3]);
  }
}

__global__ void __launch_bounds__(AD_THREADS, 2)
attention_decode_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const DecodeParams P) {
  extern __shared__ unsigned char ad_dyn[];
  unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)ad_dyn + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = ring + AD_STAGES * AD_STAGE_BYTES;       // [half][16 rows][128 bytes], swizzled
  float* merge = reinterpret_cast<float*>(q_s + AD_Q_BYTES);    // one warp's partial result: [16][HEAD_DIM + 2]
  __shared__ uint64_t full_bar[AD_STAGES], empty_bar[AD_STAGES], q_full, q_empty, item_full[AD_QUEUE], item_empty[AD_QUEUE];
  __shared__ Item item_s[AD_QUEUE];
  __shared__ int chunk_prefix[AD_MAX_SEQS + 1];
  __shared__ int s_flag;
  __shared__ int abort_flag;

  int* scan = reinterpret_cast<int*>(merge);                    // [AD_THREADS], before the first item only
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = P.group;
  int CH = P.chunk_tiles;
  if (threadIdx.x == 0) {
    const int np = AD_TILE / P.box_rows < 4 ? AD_TILE / P.box_rows : 4;   // producer warps with work
    for (int s = 0; s < AD_STAGES; ++s) { tc_mbar_init(&full_bar[s], np); tc_mbar_init(&empty_bar[s], 4); }
    tc_mbar_init(&q_full, 1);
    tc_mbar_init(&q_empty, 4);
    for (int i = 0; i < AD_QUEUE; ++i) { tc_mbar_init(&item_full[i], 1); tc_mbar_init(&item_empty[i], 4 + np - 1); }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();

  // ---- chunks of every request, and their prefix sum
  auto key_range = [&](int seq, int& tok0, int& ntok, int& ctx, int& tile_begin, int& tile_end) -> bool {
    tok0 = P.cu_tokens[seq];
    ntok = P.cu_tokens[seq + 1] - tok0;
    ctx = P.context_lens[seq];
    const int rows = ntok * G;
    if (rows <= 0 || rows > 16 || ctx <= 0) return false;
    const int pos_first = ctx - ntok, pos_last = ctx - 1;
    const int key_lo = (P.window > 0 && pos_first - P.window + 1 > 0) ? pos_first - P.window + 1 : 0;
    tile_begin = key_lo / AD_TILE;
    tile_end = pos_last / AD_TILE + 1;
    return true;
  };
  {
    const int span = (P.S + AD_THREADS - 1) / AD_THREADS;
    const int s_lo = threadIdx.x * span, s_hi = min(P.S, s_lo + span);
    // The host chose chunk_tiles for requests as long as the block table allows (a captured step is replayed while
    // its requests grow).  What the requests hold NOW decides better: the same rule as ops.attention_decode_plan,
    // on the longest request of this step, within the room the host reserved for partial results.
    if (AD_ADAPTIVE) {
      int longest = 0, count = 0, total = 0;
      for (int seq = s_lo; seq < s_hi; ++seq) {
        int tok0, ntok, ctx, tb, te;
        if (key_range(seq, tok0, ntok, ctx, tb, te)) { longest = max(longest, te - tb); ++count; total += te - tb; }
      }
      // over the block: shuffles inside a warp, then eight numbers through shared memory
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) {
        longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, o2));
        count += __shfl_xor_sync(0xffffffffu, count, o2);
        total += __shfl_xor_sync(0xffffffffu, total, o2);
      }
      if (lane == 0) { scan[warp] = longest; scan[8 + warp] = count; scan[24 + warp] = total; }
      __syncthreads();
      int tiles = 0, few = 0, sum = 0;
#pragma unroll
      for (int w = 0; w < AD_THREADS / 32; ++w) { tiles = max(tiles, scan[w]); few += scan[8 + w]; sum += scan[24 + w]; }
      // The rule takes every request for as long as the longest: it is applied where that is nearly so (the mean at
      // least 0.8 of the longest).  Requests of mixed lengths fill one another's gaps, and the host's cut was measured
      // as good or better there (56 requests of 128 to 2,300 keys: 70 us with chunks of 22 tiles, 71 us whole).
      // Thread t tries p = fewest chunks + t chunks per request; the cheapest wins, the longer chunk on a tie.
      int key = 0x7fffffff;
      if (tiles > 0 && few > 0 && (long)sum * 5 >= (long)tiles * few * 4) {
        const long cap = P.scratch_chunks / few;                       // chunks a request may have
        const int p_hi = (int)min((long)min(AD_MAX_CHUNKS, tiles), cap);
        const int p = (tiles + 63) / 64 + (int)threadIdx.x;
        if (p <= p_hi) {
          const int chunk = (tiles + p - 1) / p;
          if ((tiles + chunk - 1) / chunk == p) {
            const long rounds = ((long)few * P.n_kv * p + gridDim.x - 1) / gridDim.x;
            const long cost = rounds * (chunk + 5) * 10 + (p > 1 ? 3 * p : 0);
            if (cost < (1L << 23)) key = (int)((cost << 7) | (64 - chunk));
          }
        }
      }
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) key = min(key, __shfl_xor_sync(0xffffffffu, key, o2));
      if (lane == 0) scan[16 + warp] = key;
      __syncthreads();
#pragma unroll
      for (int w = 0; w < AD_THREADS / 32; ++w) key = min(key, scan[16 + w]);
      if (key != 0x7fffffff) CH = 64 - (key & 127);
      __syncthreads();                                           // scan is used again below
    }
    int mine = 0;
    for (int seq = s_lo; seq < s_hi; ++seq) {
      int tok0, ntok, ctx, tb, te;
      int n = key_range(seq, tok0, ntok, ctx, tb, te) ? (te - tb + CH - 1) / CH : 0;
      if (n > AD_MAX_CHUNKS || (n > 0 && (tok0 < 0 || tok0 + ntok > P.T))) {
        // more chunks than the merge takes, or tokens outside the step: the request is skipped and reported
        report_error(P.err, PHOTON_DEV_BAD_SLOT, seq, n, tok0);
        n = 0;
      }
      chunk_prefix[seq + 1] = n;                                 // counts first, sums below
      mine += n;
    }
    scan[threadIdx.x] = mine;
    __syncthreads();
    for (int off = 1; off < AD_THREADS; off <<= 1) {             // inclusive scan of the threads' totals
      const int v = threadIdx.x >= off ? scan[threadIdx.x - off] : 0;
      __syncthreads();
      scan[threadIdx.x] += v;
      __syncthreads();
    }
    int run = threadIdx.x ? scan[threadIdx.x - 1] : 0;
    if (threadIdx.x == 0) chunk_prefix[0] = 0;
    for (int seq = s_lo; seq < s_hi; ++seq) { run += chunk_prefix[seq + 1]; chunk_prefix[seq + 1] = run; }
    __syncthreads();
  }
  const int total_chunks = chunk_prefix[P.S];
  const long total_items = (long)total_chunks * P.n_kv;
  if (total_chunks > P.scratch_chunks) {
    if (threadIdx.x == 0 && blockIdx.x == 0) report_error(P.err, PHOTON_DEV_BAD_SLOT, -1, total_chunks, (int)P.scratch_chunks);
    return;
  }
  // Items are drawn from a counter by the producer, which hands them to the consumers through a small queue:
  // a block that drew short items draws more of them.  Which block computes an item changes nothing in its
  // result, and chunks are merged in chunk order.
  int* work = P.tickets + (size_t)P.S * P.n_kv;                  // [0] items handed out, [1] blocks that are done
  auto decode_item = [&](long item) -> Item {
    Item it;
    const int q_chunk = (int)(item / P.n_kv);
    it.g = (int)(item - (long)q_chunk * P.n_kv);
    int lo_s = 0, hi_s = P.S;                                    // chunk_prefix[lo_s] <= q_chunk < chunk_prefix[hi_s]
    while (hi_s - lo_s > 1) {
      const int mid = (lo_s + hi_s) >> 1;
      if (chunk_prefix[mid] <= q_chunk) lo_s = mid; else hi_s = mid;
    }
    it.seq = lo_s;
    it.chunk = q_chunk - chunk_prefix[lo_s];
    it.nchunks = chunk_prefix[lo_s + 1] - chunk_prefix[lo_s];
    int tb, te;
    key_range(it.seq, it.tok0, it.ntok, it.ctx, tb, te);
    const int pos_first = it.ctx - it.ntok;
    it.pos_last = it.ctx - 1;
    it.key_lo = (P.window > 0 && pos_first - P.window + 1 > 0) ? pos_first - P.window + 1 : 0;
    it.tile_begin = tb + it.chunk * CH;
    it.ntiles = min(te, it.tile_begin + CH) - it.tile_begin;
    return it;
  };

  const int parts = AD_TILE / P.box_rows;                        // page parts of a tile: 8, 4, 2 or 1
  const int nprod = parts < 4 ? parts : 4;                       // producer warps with work
  if (warp >= 4) {
    // ------------------------------------------------------------------ producers: Q rows and K/V tiles by TMA
    // A TMA instruction costs its issuing thread some 150 to 200 cycles, and a tile of 64 keys in pages of 16 is
    // 8 or 16 of them: one issuing thread would bound the block at 18 GB/s.  Four warps issue a page part each.
    // They give most of their registers to the consumers.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    const int pw = warp - 4;
    if (pw >= nprod) return;
    const bool leader = pw == 0;                                 // draws the items and brings Q
    const int ppw = (parts + 3) / 4;                             // parts of this warp per tile: pw, pw + 4
    uint32_t n = 0;                                              // tiles issued so far: stage and parity follow
    uint32_t items = 0;
    AD_T(long long t_wait = 0; const long long t_begin = clock64();)
    for (;; ++items) {
      const int qs = (int)(items % AD_QUEUE);
      int ok = 1;
      if (leader) {
        long item = 0;
        if (lane == 0) {
          ok = tc_wait(&item_empty[qs], ((items / AD_QUEUE) & 1u) ^ 1u, &abort_flag) ? 1 : 0;
          item = ok ? (long)atomicAdd(work, 1) : total_items;
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        item = __shfl_sync(0xffffffffu, item, 0);
        if (item >= total_items) {
          if (lane == 0 && ok) { item_s[qs].ntiles = -1; tc_mbar_arrive(&item_full[qs]); }
          break;
        }
        const Item mine = decode_item(item);
        if (lane == 0) { item_s[qs] = mine; tc_mbar_arrive(&item_full[qs]); }    // arrive releases the writes before it
        __syncwarp();
      } else {
        if (lane == 0) ok = tc_wait(&item_full[qs], (items / AD_QUEUE) & 1u, &abort_flag) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
      }
      const Item it = item_s[qs];
      __syncwarp();
      if (!leader && lane == 0) tc_mbar_arrive(&item_empty[qs]);
      if (it.ntiles < 0) break;
      if (leader && lane == 0) {
        ok = tc_wait(&q_empty, (items & 1u) ^ 1u, &abort_flag) ? 1 : 0;      // the consumers have the last item's Q in registers
        if (ok) {
          tc_mbar_expect_tx(&q_full, (uint32_t)P.q_rows * 128u * AD_DH);
#pragma unroll
          for (int h = 0; h < AD_DH; ++h) tc_tma_load3(q_s + h * (16 * 128), &map_q, h * 64, it.g * G, it.tok0, &q_full);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      // the pages of this warp's parts: lane j holds those of tiles j and j + 32 (an item has at most 64 tiles)
      const int* table = P.block_table + (size_t)it.seq * P.max_pages;
      int page_of[2][2];
#pragma unroll
      for (int pp = 0; pp < 2; ++pp)
#pragma unroll
        for (int hi = 0; hi < 2; ++hi) {
          const int i = lane + 32 * hi;
          const int key = (it.tile_begin + i) * AD_TILE + (pw + 4 * pp) * P.box_rows;
          const int pidx = key / P.page_size;
          page_of[pp][hi] = (pp < ppw && i < it.ntiles && pidx < P.max_pages && key <= it.pos_last &&
                             key + P.box_rows - 1 >= it.key_lo) ? table[pidx] : -2;       // -2: not needed
        }
      for (int i = 0; i < it.ntiles; ++i, ++n) {
        const int s = (int)(n % AD_STAGES);
        int rowc[2];
#pragma unroll
        for (int pp = 0; pp < 2; ++pp) {
          const int page = __shfl_sync(0xffffffffu, i < 32 ? page_of[pp][0] : page_of[pp][1], i & 31);
          const int key = (it.tile_begin + i) * AD_TILE + (pw + 4 * pp) * P.box_rows;
          rowc[pp] = P.total_rows;                               // outside the map: the part is filled with zeros
          if (page >= 0 && page < P.num_pages) rowc[pp] = (page * P.n_kv + it.g) * P.page_size + (key % P.page_size);
          else if (page != -2 && lane == 0) report_error(P.err, PHOTON_DEV_BAD_PAGE, it.tok0, key, page);
        }
        if (lane == 0) {
          AD_T(const long long t0 = clock64();)
          ok = tc_wait(&empty_bar[s], ((n / AD_STAGES) & 1u) ^ 1u, &abort_flag) ? 1 : 0;
          AD_T(t_wait += clock64() - t0;)
          if (ok) {
            tc_mbar_expect_tx(&full_bar[s], (uint32_t)(ppw * P.box_rows * 128 * AD_DH * 2));
            for (int pp = 0; pp < ppw; ++pp) {
              unsigned char* kst = ring + (size_t)s * AD_STAGE_BYTES + (pw + 4 * pp) * P.box_rows * 128;
#pragma unroll
              for (int h = 0; h < AD_DH; ++h) tc_tma_load(kst + h * AD_HALF_BYTES, &map_k, h * 64, rowc[pp], &full_bar[s]);
#pragma unroll
              for (int h = 0; h < AD_DH; ++h) tc_tma_load(kst + AD_KV_BYTES + h * AD_HALF_BYTES, &map_v, h * 64, rowc[pp], &full_bar[s]);
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
      }
      if (!ok) break;
    }
    AD_T(if (leader && lane == 0 && blockIdx.x == 0) { ad_trace[0] = t_wait; ad_trace[1] = clock64() - t_begin; })
    if (leader && lane == 0) {
      // the block that is done last puts both counters back to zero for the next launch
      __threadfence();
      if (atomicAdd(work + 1, 1) == (int)gridDim.x - 1) { work[0] = 0; work[1] = 0; }
    }
    if (lane == 0 && abort_flag) {
      // copies already started still write into this block's shared memory: wait for them, bounded
      for (uint32_t j = (n > AD_STAGES ? n - AD_STAGES : 0); j < n; ++j)
        for (uint32_t w = 0; w < TC_WAIT_LIMIT && !tc_mbar_try(&full_bar[j % AD_STAGES], (j / AD_STAGES) & 1u); ++w) {}
      for (uint32_t w = 0; leader && items > 0 && w < TC_WAIT_LIMIT && !tc_mbar_try(&q_full, (items - 1) & 1u); ++w) {}
      if (leader) report_error(P.err, PHOTON_DEV_WAIT_TIMEOUT, 30, blockIdx.x, 0);
    }
    return;
  }

  asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
  // -------------------------------------------------------------------- consumers: four warps, 16 keys of every tile each
  auto consumer_sync = [&]() { asm volatile("bar.sync 1, 128;" ::: "memory"); };
  const uint32_t ring_addr = tc_smem(ring), q_addr = tc_smem(q_s);
  uint32_t n = 0, items = 0;
  bool alive = true;
  AD_T(long long c_wait = 0, c_tiles = 0, c_merge = 0; const long long c_begin = clock64();)
  for (;; ++items) {
    const int qs = (int)(items % AD_QUEUE);
    if (alive && !tc_wait(&item_full[qs], (items / AD_QUEUE) & 1u, &abort_flag)) alive = false;
    consumer_sync();
    if (abort_flag) break;                                       // the four warps read the same flag after the same barrier
    const Item it = item_s[qs];
    __syncwarp();
    if (lane == 0) tc_mbar_arrive(&item_empty[qs]);
    if (it.ntiles < 0) break;
    const int rows = it.ntok * G;
    int pos_r[2], lo_r[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      const int row = (lane >> 2) + h2 * 8;
      if (row < rows) {
        pos_r[h2] = it.ctx - it.ntok + row / G;
        lo_r[h2] = (P.window > 0 && pos_r[h2] - P.window + 1 > 0) ? pos_r[h2] - P.window + 1 : 0;
      } else {
        pos_r[h2] = -1; lo_r[h2] = 0;                            // a row of the box that is not this request's: sees nothing
      }
    }
    int warp_pos_max = max(pos_r[0], pos_r[1]), warp_pos_min = min(pos_r[0], pos_r[1]), warp_lo_max = max(lo_r[0], lo_r[1]);
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) {
      warp_pos_max = max(warp_pos_max, __shfl_xor_sync(0xffffffffu, warp_pos_max, o2));
      warp_pos_min = min(warp_pos_min, __shfl_xor_sync(0xffffffffu, warp_pos_min, o2));
      warp_lo_max = max(warp_lo_max, __shfl_xor_sync(0xffffffffu, warp_lo_max, o2));
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[AD_ND][4];
#pragma unroll
    for (int nn = 0; nn < AD_ND; ++nn) { o[nn][0] = o[nn][1] = o[nn][2] = o[nn][3] = 0.f; }
    uint32_t qa[AD_KD][4];
    if (alive && !tc_wait(&q_full, items & 1u, &abort_flag)) alive = false;
#pragma unroll
    for (int kd = 0; kd < AD_KD; ++kd) {
      // A fragment of the 16 query rows: row lane % 16, features kd * 16 + 8 * (lane / 16)
      const int row = lane & 15, dim = kd * 16 + ((lane >> 4) << 3);
      ad_ldsm4(qa[kd], q_addr + (uint32_t)((dim >> 6) * (16 * 128) + row * 128 + ((((dim & 63) >> 3) ^ (row & 7)) << 4)));
    }
    __syncwarp();
    if (lane == 0 && alive) tc_mbar_arrive(&q_empty);            // Q is in registers

    for (int i = 0; i < it.ntiles; ++i, ++n) {
      const int s = (int)(n % AD_STAGES);
      AD_T(const long long t0 = clock64();)
      if (alive && !tc_wait(&full_bar[s], (n / AD_STAGES) & 1u, &abort_flag)) alive = false;
      AD_T(const long long t1 = clock64(); c_wait += t1 - t0;)
      const int key_base = (it.tile_begin + i) * AD_TILE;
      const uint32_t ks = ring_addr + (uint32_t)s * AD_STAGE_BYTES, vs = ks + AD_KV_BYTES;
      if (key_base < it.key_lo || key_base + AD_TILE - 1 > it.pos_last) {
        // value rows outside the visible range: zeros (uniform for the block: first and last tiles only)
        unsigned char* vst = ring + (size_t)s * AD_STAGE_BYTES + AD_KV_BYTES;
        for (int c = threadIdx.x; c < AD_TILE * (HEAD_DIM / 8); c += 128) {
          const int r = c / (HEAD_DIM / 8), piece = c - r * (HEAD_DIM / 8);
          const int key = key_base + r;
          if (key < it.key_lo || key > it.pos_last)
            *reinterpret_cast<uint4*>(vst + (piece >> 3) * AD_HALF_BYTES + r * 128 + ((piece & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // before a later TMA write to this stage
        consumer_sync();
      }
      const int k0 = key_base + warp * 16;
      if (alive && k0 <= warp_pos_max) {
        if (k0 + 15 <= warp_pos_min && k0 >= warp_lo_max)
          ad_warp_tile<false>(qa, ks, vs, warp * 16, key_base, pos_r[0], pos_r[1], lo_r[0], lo_r[1], P.scale_log2, m, l, o);
        else
          ad_warp_tile<true>(qa, ks, vs, warp * 16, key_base, pos_r[0], pos_r[1], lo_r[0], lo_r[1], P.scale_log2, m, l, o);
      }
      __syncwarp();
      if (lane == 0 && alive) tc_mbar_arrive(&empty_bar[s]);     // this warp is done with the stage
      AD_T(c_tiles += clock64() - t1;)
    }
    AD_T(const long long t2 = clock64();)

    // ---- the quad's partial sums, then the four warps merged into warp 0: 3 into 2, 2 into 1, 1 into 0
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      l[h2] += __shfl_xor_sync(0xffffffffu, l[h2], 1);
      l[h2] += __shfl_xor_sync(0xffffffffu, l[h2], 2);
    }
    constexpr int MLD = HEAD_DIM + 2;                            // a row: HEAD_DIM sums, then max and sum
    for (int src = 3; src >= 1; --src) {
      if (warp == src) {
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          float* row = merge + ((lane >> 2) + h2 * 8) * MLD;
          if ((lane & 3) == 0) { row[HEAD_DIM] = m[h2]; row[HEAD_DIM + 1] = l[h2]; }
#pragma unroll
          for (int nn = 0; nn < AD_ND; ++nn)
            *reinterpret_cast<float2*>(row + nn * 8 + (lane & 3) * 2) = make_float2(o[nn][h2 * 2], o[nn][h2 * 2 + 1]);
        }
      }
      consumer_sync();
      if (warp == src - 1) {
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          const float* row = merge + ((lane >> 2) + h2 * 8) * MLD;
          const float m2 = row[HEAD_DIM], l2 = row[HEAD_DIM + 1];
          const float M = fmaxf(m[h2], m2);
          const float a = (m[h2] == -INFINITY) ? 0.f : exp2f(m[h2] - M), b = (m2 == -INFINITY) ? 0.f : exp2f(m2 - M);
          m[h2] = M;
          l[h2] = l[h2] * a + l2 * b;
#pragma unroll
          for (int nn = 0; nn < AD_ND; ++nn) {
            const float2 v = *reinterpret_cast<const float2*>(row + nn * 8 + (lane & 3) * 2);
            o[nn][h2 * 2] = o[nn][h2 * 2] * a + v.x * b;
            o[nn][h2 * 2 + 1] = o[nn][h2 * 2 + 1] * a + v.y * b;
          }
        }
      }
      consumer_sync();
    }
    // warp 0 holds the item's result: (m, l, o) of the 16 rows
    const size_t part = ((size_t)(chunk_prefix[it.seq] + it.chunk) * P.n_kv + it.g) * 16;   // this item's rows in the scratch
    if (warp == 0) {
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const int r = (lane >> 2) + h2 * 8;
        if (r >= rows) continue;
        if (it.nchunks == 1) {
          const int tk = r / G, h = r - tk * G;
          const float inv = l[h2] > 0.f ? 1.f / l[h2] : 0.f;
          bf16* dst = P.out + (size_t)(it.tok0 + tk) * P.out_stride + (size_t)(it.g * G + h) * HEAD_DIM + (lane & 3) * 2;
#pragma unroll
          for (int nn = 0; nn < AD_ND; ++nn)
            *reinterpret_cast<__nv_bfloat162*>(dst + nn * 8) = __floats2bfloat162_rn(o[nn][h2 * 2] * inv, o[nn][h2 * 2 + 1] * inv);
        } else {
          float* acc = P.part_acc + (part + r) * HEAD_DIM + (lane & 3) * 2;
#pragma unroll
          for (int nn = 0; nn < AD_ND; ++nn) __stcg(reinterpret_cast<float2*>(acc + nn * 8), make_float2(o[nn][h2 * 2], o[nn][h2 * 2 + 1]));
          if ((lane & 3) == 0) { __stcg(P.part_ml + (part + r) * 2, m[h2]); __stcg(P.part_ml + (part + r) * 2 + 1, l[h2]); }
        }
      }
    }
    if (it.nchunks > 1) {
      // the block that draws the last ticket of (request, key/value head) merges the chunks in chunk order
      __threadfence();
      consumer_sync();
      if (threadIdx.x == 0) s_flag = (atomicAdd(P.tickets + (size_t)it.seq * P.n_kv + it.g, 1) == it.nchunks - 1);
      consumer_sync();
      if (s_flag) {
        __threadfence();
        if (threadIdx.x == 0) P.tickets[(size_t)it.seq * P.n_kv + it.g] = 0;
        // first the chunks' maxima and sums: warp w takes rows w, w + 4, ..., a lane up to four chunks (one round
        // trip); every chunk's weight 2^(m_c - M) goes to shared memory (the merge buffer is free), the row's
        // 1 / sum with it
        float* weight = merge;                                   // [rows][nchunks], then [rows] reciprocal sums
        const size_t base = (size_t)chunk_prefix[it.seq] * P.n_kv + it.g;
        for (int r = warp; r < rows; r += 4) {
          float2 ml[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = lane + 32 * j;
            ml[j] = c < it.nchunks ? __ldcg(reinterpret_cast<const float2*>(P.part_ml + (((base + (size_t)c * P.n_kv) * 16) + r) * 2))
                                   : make_float2(-INFINITY, 0.f);
          }
          const float M = warp_max(fmaxf(fmaxf(ml[0].x, ml[1].x), fmaxf(ml[2].x, ml[3].x)));
          float L = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = lane + 32 * j;
            const float sc = (ml[j].x == -INFINITY || M == -INFINITY) ? 0.f : exp2f(ml[j].x - M);
            if (c < it.nchunks) weight[r * it.nchunks + c] = sc;
            L += ml[j].y * sc;
          }
          // lanes hold chunks c, c + 32, ...: added in a fixed order (lane's own, then the shuffle tree)
          L = warp_sum(L);
          if (lane == 0) weight[rows * it.nchunks + r] = L > 0.f ? 1.f / L : 0.f;
        }
        consumer_sync();
        // then the weighted sums: a thread takes four neighbouring features of a row; the chunks' loads do not
        // depend on one another
        for (int e = threadIdx.x * 4; e < rows * HEAD_DIM; e += 128 * 4) {
          const int r = e / HEAD_DIM, d = e - r * HEAD_DIM;
          const float* w = weight + r * it.nchunks;
          const float* acc = P.part_acc + ((base * 16) + r) * HEAD_DIM + d;
          const size_t step = (size_t)P.n_kv * 16 * HEAD_DIM;
          float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
          int c = 0;
          for (; c + 4 <= it.nchunks; c += 4) {
            float4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = __ldcg(reinterpret_cast<const float4*>(acc + (size_t)(c + j) * step));
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float wj = w[c + j];
              A.x += v[j].x * wj; A.y += v[j].y * wj; A.z += v[j].z * wj; A.w += v[j].w * wj;
            }
          }
          for (; c < it.nchunks; ++c) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(acc + (size_t)c * step));
            const float wj = w[c];
            A.x += v.x * wj; A.y += v.y * wj; A.z += v.z * wj; A.w += v.w * wj;
          }
          const float inv = weight[rows * it.nchunks + r];
          const int tk = r / G, h = r - tk * G;
          bf16* dst = P.out + (size_t)(it.tok0 + tk) * P.out_stride + (size_t)(it.g * G + h) * HEAD_DIM + d;
          *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(A.x * inv, A.y * inv);
          *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(A.z * inv, A.w * inv);
        }
      }
      consumer_sync();                                           // s_flag is free for the next item
    }
    AD_T(c_merge += clock64() - t2;)
  }
  AD_T(if (threadIdx.x == 0 && blockIdx.x == 0) { ad_trace[2] = c_wait; ad_trace[3] = c_tiles; ad_trace[4] = c_merge;
                                                   ad_trace[5] = clock64() - c_begin; ad_trace[6] = n; ad_trace[7] = items; })
  pdl_launch_dependents();
}

// ---------------------------------------------------------------------------------------------------- host
PHOTON_API int photon_attention_decode_head_dim() { return HEAD_DIM; }

// Blocks of the kernel that the current device holds at once (its grid).
PHOTON_API int photon_attention_decode_slots() {
  static int slots = 0;
  if (slots == 0) {
    cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AD_SMEM_BYTES);
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_kernel, AD_THREADS, AD_SMEM_BYTES) != cudaSuccess ||
        per_sm <= 0) {
      cudaGetLastError();
      per_sm = 1;
    }
    slots = per_sm * photon_sm_count();
  }
  return slots;
}

// Attention of the requests of the step that bring at most 16 rows (tokens x group); the others are left
// untouched.  q [T, n_q * d] with row stride q_stride, out [T, n_q * d]; k_cache, v_cache [num_pages, n_kv,
// page_size, d] contiguous; page_size a multiple of 8 that divides 64 or is a multiple of 64; S <= 512.
// chunk_tiles: tiles of 64 keys per work item (1..64); max_chunks_per_seq: what the longest request then has (<= 120).  part_acc (float, scratch_chunks * n_kv * 16 * d),
// part_ml (float, scratch_chunks * n_kv * 32): partial results of requests with more than one chunk;
// scratch_chunks must be at least the chunks of all requests together.  tickets: int [S * n_kv], all zero
// between launches.  T: tokens of the step (rows of q).  max_items: an upper bound of the work items (sizes the grid; 0: as many blocks as fit).
PHOTON_API int photon_attention_decode(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                                       const void* v_cache, const int* block_table, int max_pages, const int* cu_tokens,
                                       const int* context_lens, float* part_acc, float* part_ml, long scratch_chunks,
                                       int* tickets, int S, int T, int n_q, int n_kv, int d, int page_size, int num_pages,
                                       int window, float scale, int chunk_tiles, int max_chunks_per_seq, long max_items, int* err,
                                       cudaStream_t stream) {
  if (S <= 0) return 0;
  if (d != HEAD_DIM || n_kv <= 0 || n_q % n_kv || !(scale > 0.f) || S > AD_MAX_SEQS) return PHOTON_ERR_UNSUPPORTED;
  if (n_q / n_kv > 16 || chunk_tiles < 1 || chunk_tiles > 64) return PHOTON_ERR_UNSUPPORTED;
  if (page_size < 8 || (page_size & 7) || !((AD_TILE % page_size) == 0 || (page_size % AD_TILE) == 0)) return PHOTON_ERR_UNSUPPORTED;
  if (max_chunks_per_seq < 1 || max_chunks_per_seq > AD_MAX_CHUNKS) return PHOTON_ERR_UNSUPPORTED;
  if (((uintptr_t)q & 15) || (q_stride & 7) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) ||
      context_lens == nullptr || cu_tokens == nullptr || tickets == nullptr || part_acc == nullptr || part_ml == nullptr)
    return PHOTON_ERR_ARGUMENT;
  const long total_rows = (long)num_pages * n_kv * page_size;
  if (total_rows > 0x7fffffffL) return PHOTON_ERR_UNSUPPORTED;
  const int box_rows = page_size < AD_TILE ? page_size : AD_TILE;
  CUtensorMap map_q, map_k, map_v;
  const int G = n_q / n_kv;
  {
    // Q as [T][n_q][d]: a box holds the GROUP heads of floor(16 / GROUP) tokens, 64 features wide
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return PHOTON_ERR_UNSUPPORTED;
    cuuint64_t dims[3] = {(cuuint64_t)d, (cuuint64_t)n_q, (cuuint64_t)T};
    cuuint64_t strides[2] = {(cuuint64_t)d * 2, (cuuint64_t)q_stride * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(16 / G)};
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
  DecodeParams P;
  P.q = (const bf16*)q; P.q_stride = q_stride; P.out = (bf16*)out; P.out_stride = out_stride;
  P.block_table = block_table; P.max_pages = max_pages; P.cu_tokens = cu_tokens; P.context_lens = context_lens;
  P.part_acc = part_acc; P.part_ml = part_ml; P.scratch_chunks = scratch_chunks; P.tickets = tickets;
  P.q_rows = G * (16 / G);
  P.T = T;
  P.S = S; P.n_kv = n_kv; P.group = G; P.page_size = page_size; P.num_pages = num_pages;
  P.total_rows = (int)total_rows; P.box_rows = box_rows; P.window = window; P.chunk_tiles = chunk_tiles;
  P.scale_log2 = scale * 1.4426950408889634f; P.err = err;
  const int slots = photon_attention_decode_slots();
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  const long grid = slots;                          // blocks without an item leave at once; the kernel may cut finer than the host
  return launch_pdl(attention_decode_kernel, dim3((unsigned)grid), dim3(AD_THREADS), (size_t)AD_SMEM_BYTES, stream, map_q, map_k, map_v, P);
}
