/* photon/kernels.h: the C interface of the sm_100a kernels of photon_infer_b200.
 *
 * Every kernel source under csrc/ becomes one shared library; the functions below are what those libraries
 * export (C linkage, default visibility).  The Python side (photon_infer_b200/kernels/ops.py) calls them through
 * ctypes; a C or C++ program can link the libraries and call them the same way.  csrc/common.cuh includes this
 * header, so a definition that drifts from its declaration does not compile.
 *
 * lumia431/photon_infer's library surface is C++ classes (include/photon/arch/llama_model.hpp:61-240,
 * include/photon/scheduler/continuous_batch_engine.hpp:48-315).  Here the host side (configuration, weights,
 * cache manager, step function, scheduler) is Python; this header is the part of the library that is native.
 *
 * Conventions
 *   - All pointers are device pointers unless a comment says "host".  Kernels run on `stream`.
 *   - Return value: 0 = launched; > 0 = a cudaError_t; PHOTON_ERR_UNSUPPORTED (-2) = this size or alignment is
 *     refused (nothing ran); PHOTON_ERR_ARGUMENT (-3) = invalid argument.  Never a wrong result.
 *   - dtype codes: PHOTON_F32 0, PHOTON_BF16 1.
 *   - `err`: int[4] on the device (may be null).  A kernel that meets a bad index (token id, cache slot, page)
 *     skips the access and records {code, detail0, detail1, detail2} once (PHOTON_DEV_* below); a bounded wait
 *     that ran out records PHOTON_DEV_WAIT_TIMEOUT.
 *   - The paged cache of one layer: K and V each [num_pages][n_kv][page_size][head_dim], contiguous.
 *     block_table [S][max_pages] int: pages of request s in order, -1 where none is held.
 *     slot_mapping [T] int: page * page_size + offset of each token of the step; -1 = do not store.
 *   - A step holds T tokens of S requests; cu_tokens [S + 1] gives each request's first token;
 *     positions [T] each token's position in its request; a token at position p sees keys max(0, p - window + 1)..p
 *     (window 0: all keys up to p).
 *   - Matrix products compute out[M, N] = x[M, K] * W[N, K]^T (W row-major [out, in], no bias), leading
 *     dimensions in elements.
 */
#ifndef PHOTON_KERNELS_H
#define PHOTON_KERNELS_H

#include <cuda_runtime.h>

#if defined(__GNUC__)
#define PHOTON_EXPORT __attribute__((visibility("default")))
#else
#define PHOTON_EXPORT
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define PHOTON_F32 0
#define PHOTON_BF16 1
#define PHOTON_ERR_UNSUPPORTED (-2)
#define PHOTON_ERR_ARGUMENT (-3)
#define PHOTON_DEV_BAD_TOKEN 1
#define PHOTON_DEV_BAD_SLOT 2
#define PHOTON_DEV_BAD_PAGE 3
#define PHOTON_DEV_WAIT_TIMEOUT 4

/* ------------------------------------------------------------------ elementwise.cu */
/* out[t, :] = table[ids[t], :] as float; ids outside [0, V) give a zero row and PHOTON_DEV_BAD_TOKEN. */
PHOTON_EXPORT int photon_embedding(const int* ids, const void* table, int table_dtype, float* out, int T, int H, int V, int* err,
                     cudaStream_t stream);
/* residual (float [*, H], in place) += delta; out = w * residual / sqrt(mean(residual^2) + eps).  delta may be null.
 * rows (may be null): only these rows are read, nothing is written back, out has one row per entry. */
PHOTON_EXPORT int photon_add_rmsnorm(const void* delta, int delta_dtype, float* residual, const void* w, int w_dtype, void* out,
                       int out_dtype, const int* rows, int n, int H, float eps, cudaStream_t stream);
/* out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]; gate_up [T, 2I], out [T, I] of one dtype. */
PHOTON_EXPORT int photon_swiglu(const void* gate_up, void* out, int dtype, int T, int I, cudaStream_t stream);

/* ------------------------------------------------------------------ rope_kv.cu */
/* Rotates q [T, n_q * d] and k [T, n_kv * d] in place (rotate != 0; pairs (2j, 2j+1) when interleaved, else
 * (j, j + d/2); angle positions[t] * inv_freq[j] in 32-bit) and stores k, v at slot_mapping in the cache
 * (write_kv != 0).  q, k, v may be views with any row stride (elements). */
PHOTON_EXPORT int photon_rope_kv_write(void* q, long q_stride, void* k, long k_stride, const void* v, long v_stride, int dtype,
                         const int* positions, const float* inv_freq, int interleaved, const int* slot_mapping,
                         void* k_cache, void* v_cache, int T, int n_q, int n_kv, int d, int page_size, long num_slots,
                         int rotate, int write_kv, int* err, cudaStream_t stream);
/* out [count][half][2] float: (cos, sin) of position * inv_freq[j]. */
PHOTON_EXPORT int photon_rope_table(const float* inv_freq, int half, int count, void* out, cudaStream_t stream);

/* ------------------------------------------------------------------ attention.cu (float32 and any even head size) */
PHOTON_EXPORT int photon_paged_attention(const void* q, long q_stride, void* out, long out_stride, int dtype, const void* k_cache,
                           const void* v_cache, const int* block_table, int max_pages, const int* token_seq,
                           const int* positions, int T_, int n_q, int n_kv, int d, int page_size, int num_pages,
                           int window, float scale, int* err, cudaStream_t stream);

/* ------------------------------------------------------------------ attention_flash.cu (-DHEAD_DIM=d, d % 16 == 0, <= 128; bfloat16) */
PHOTON_EXPORT int photon_flash_attention_head_dim(void);
PHOTON_EXPORT int photon_flash_attention_max_groups(void);
/* mode bit 0: requests with more than 16 rows (tokens x heads per key/value head); bit 1: the others, their keys
 * split over num_splits blocks (part_acc/part_ml: float scratch of T * n_q * num_splits * (d + 2); tickets: int
 * [S * n_kv], zero between launches) and over nsub groups of warps per block.  context_lens may be null. */
PHOTON_EXPORT int photon_flash_attention(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                           const void* v_cache, const int* block_table, int max_pages, const int* cu_tokens,
                           const int* positions, const int* context_lens, float* part_acc, float* part_ml, int* tickets,
                           int S, int max_tokens_per_seq, int n_q, int n_kv, int d, int page_size, int num_pages,
                           int window, float scale, int num_splits, int nsub, int mode, int* err, cudaStream_t stream);

/* ------------------------------------------------------------------ attention_tc.cu (-DHEAD_DIM=64|128; bfloat16; tcgen05) */
PHOTON_EXPORT int photon_attention_tc_head_dim(void);
/* Requests with more than 16 rows only; the others are left untouched. */
PHOTON_EXPORT int photon_attention_tc(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                        const void* v_cache, const int* block_table, int max_pages, const int* cu_tokens,
                        const int* positions, int S, int max_tokens_per_seq, int T, int n_q, int n_kv, int d,
                        int page_size, int num_pages, int window, float scale, int* err, cudaStream_t stream);

/* ------------------------------------------------------------------ attention_decode.cu (-DHEAD_DIM=64|128; bfloat16; TMA) */
PHOTON_EXPORT int photon_attention_decode_head_dim(void);
PHOTON_EXPORT int photon_attention_decode_slots(void);           /* blocks the current device holds at once (the kernel's grid) */
/* Requests with at most 16 rows only (S <= 512).  context_lens [S]: tokens of each request after this step.
 * chunk_tiles: tiles of 64 keys per work item (1..64); max_chunks_per_seq <= 120.  part_acc: float
 * [scratch_chunks * n_kv * 16 * d], part_ml: float [scratch_chunks * n_kv * 32]; scratch_chunks >= the chunks of
 * all requests together.  tickets: int [S * n_kv + 2], zero between launches.  max_items: bound of the work
 * items (sizes the grid; 0: as many blocks as fit). */
PHOTON_EXPORT int photon_attention_decode(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                            const void* v_cache, const int* block_table, int max_pages, const int* cu_tokens,
                            const int* context_lens, float* part_acc, float* part_ml, long scratch_chunks, int* tickets,
                            int S, int T, int n_q, int n_kv, int d, int page_size, int num_pages, int window,
                            float scale, int chunk_tiles, int max_chunks_per_seq, long max_items, int* err,
                            cudaStream_t stream);

/* ------------------------------------------------------------------ gemm_f32.cu: true 32-bit product (FMA chain in ascending k) */
PHOTON_EXPORT int photon_sgemm_nt(const float* A, long lda, const float* W, long ldw, float* C, long ldc, int M, int N, int K,
                    cudaStream_t stream);

/* ------------------------------------------------------------------ gemm_skinny.cu: bfloat16, M <= 64 (32 with SwiGLU) */
/* epilogue 0: bfloat16 out; 1: float out; 2: SwiGLU (W = [gate rows; up rows], out [M, N / 2]).  K % 8 == 0,
 * 16-byte aligned rows.  scratch (float) and tickets (int, zero between launches) serve the split of K; launches
 * that share them must not overlap on the device. */
PHOTON_EXPORT int photon_skinny_gemm(const void* x, long ldx, const void* W, long ldw, void* out, long ldo, int M, int N, int K,
                       int epilogue, float* scratch, long scratch_floats, int* tickets, int num_tickets,
                       cudaStream_t stream);

/* ------------------------------------------------------------------ gemm_skinny_fused.cu: M <= 8 */
/* x = res_in + delta (res_out gets the sum when delta is given); out = epilogue(rmsnorm(x; norm_w, eps) W^T).
 * epilogue 0: bfloat16; 2: SwiGLU; 3: q/k/v with rotation (partners must be neighbouring rows of W) and cache write. */
PHOTON_EXPORT int photon_skinny_fused(const float* res_in, float* res_out, const void* delta, const void* norm_w, int norm_w_dtype,
                        float eps, const void* W, long ldw, void* out, long ldo, int M, int N, int K, int epilogue,
                        const int* positions, const float* inv_freq, const int* slot_mapping, void* k_cache,
                        void* v_cache, int n_q, int n_kv, int d, int page_size, long num_slots, int* err,
                        cudaStream_t stream);

/* ------------------------------------------------------------------ gemm_skinny_static.cu: see gemm_skinny_static.h */
PHOTON_EXPORT const char* photon_static_error_string(int code);
PHOTON_EXPORT int photon_skinny_gemm_static(const void* x, long ldx, const void* W, long ldw, void* out, long ldo, int M, int N, int K,
                              int epilogue, cudaStream_t stream);

/* ------------------------------------------------------------------ gemm_tc.cu, gemm_tc2.cu: bfloat16 on tcgen05 (TMA, tensor memory) */
/* epilogue as photon_skinny_gemm.  gemm_tc: tiles of 128 x 256 on one SM; gemm_tc2: 256 x 256 on pairs of SMs. */
PHOTON_EXPORT int photon_gemm_tc(const void* x, long ldx, const void* W, long ldw, void* out, long ldo, int M, int N, int K,
                   int epilogue, int* err, cudaStream_t stream);
PHOTON_EXPORT int photon_gemm_tc2(const void* x, long ldx, const void* W, long ldw, void* out, long ldo, int M, int N, int K,
                    int epilogue, int* err, cudaStream_t stream);
/* x W^T with W = [q; k; v] rows (rotation partners as neighbours): rotated q to q_out [M, n_q * d], rotated k and v
 * to slot_mapping of the cache.  table (may be null): photon_rope_table output of table_positions positions. */
PHOTON_EXPORT int photon_gemm_tc2_qkv(const void* x, long ldx, const void* W, long ldw, void* q_out, long ldo, int M, int K,
                        const int* positions, const int* slot_mapping, const float* inv_freq, const void* table,
                        int table_positions, void* k_cache, void* v_cache, int n_q, int n_kv, int d, int page_size,
                        long num_slots, int* err, cudaStream_t stream);

/* ------------------------------------------------------------------ sampling.cu */
/* Per row: first maximum where temperature is null or <= 0, else the first index whose running sum of
 * softmax(logits / temperature) reaches u.  scratch: float [rows * 128] for V > 16384, else may be null. */
PHOTON_EXPORT int photon_sample(const float* logits, long ld, const float* temperature, const float* u, int* out, int rows, int V,
                  float* scratch, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* PHOTON_KERNELS_H */
