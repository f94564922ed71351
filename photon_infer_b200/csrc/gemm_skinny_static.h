// photon_skinny_gemm_static: the few-rows matrix product for callers that cannot allocate.
//
// This entry point has no counterpart in lumia431/photon_infer.
//
// Who needs it: code that runs where device memory must not be requested or released: a
// plugin inside another runtime that owns the allocator, a serving loop that has promised
// its host not to call cudaMalloc on the hot path (it can stall every stream of the
// process), or a process whose device memory was handed out completely at start-up.  The
// regular entry point,
// photon_skinny_gemm, needs a scratch buffer and a ticket array from its caller when it
// splits K over several blocks; whoever calls it has to get those from somewhere.  This
// variant brings its own: one array in the library's device image, so every GPU that loads
// the library holds PHOTON_STATIC_SCRATCH_BYTES of it until the process exits.
//
// What it computes: out[M, N] = x[M, K] * W[N, K]^T in bfloat16 with 32-bit accumulation,
// with the same kernels, the same split of K and therefore the same bits as
// photon_skinny_gemm.  The caller passes inputs and outputs only.
//
// Limits (beyond them the call returns PHOTON_STATIC_TOO_LARGE and launches nothing):
//   M <= 64 (32 with the SwiGLU epilogue), N <= PHOTON_STATIC_MAX_ROWS output features,
//   K a multiple of 8, rows of x and W 16-byte aligned.
//
// Set-up: the first call on a device looks up the array's device address
// (cudaGetSymbolAddress, with that device current) and remembers it for that device.  Make
// that first call before any stream capture begins.
//
// Sharing: all calls on a device use the same array.  It keeps whatever the last call left;
// the part that has to start at zero (the tickets) is cleared on the stream at the start of
// every call.  Two calls that overlap on the GPU (different streams, or graphs replayed side
// by side) race on it: run them one after the other.
//
// It calls no cudaMalloc, cudaFree or any routine that allocates.
#pragma once
#include <cuda_runtime.h>

#define PHOTON_STATIC_MAX_ROWS 131072                      /* output features (N), 8192 row tiles */
#define PHOTON_STATIC_SHARE_FLOATS (1u << 20)              /* 4 MiB of partial sums */
#define PHOTON_STATIC_SCRATCH_BYTES (32768u + 4u * PHOTON_STATIC_SHARE_FLOATS)
#define PHOTON_STATIC_TOO_LARGE (-4)

#ifdef __cplusplus
extern "C" {
#endif

// epilogue: 0 bfloat16 output, 1 float output, 2 SwiGLU (W holds gate rows then up rows, out is [M, N/2]).
// Returns 0, a CUDA error code (> 0), PHOTON_STATIC_TOO_LARGE, or -2 / -3 for a shape or alignment the
// kernel does not take.  photon_static_error_string turns the code into words.
int photon_skinny_gemm_static(const void* x, long ldx, const void* W, long ldw, void* out, long ldo, int M, int N,
                              int K, int epilogue, cudaStream_t stream);

const char* photon_static_error_string(int code);

#ifdef __cplusplus
}
#endif
