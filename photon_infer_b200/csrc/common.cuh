// Shared helpers of the sm_100a kernels: storage types, 32-bit conversion, block
// reductions with a fixed order, the error word that kernels write on a bad index.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>

// The exported entry points, the dtype codes shared with kernels/ops.py, the launcher's return codes and the
// codes that kernels write into the error word: declared once, for C callers too.  A definition below that
// does not match its declaration there is a compile error.
#include <photon/kernels.h>

#define PHOTON_API extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Loads a weight that may be stored in either type (norm weights keep 32-bit storage).
__device__ __forceinline__ float load_w(const void* w, int is_bf16, size_t i) {
  return is_bf16 ? __bfloat162float(((const bf16*)w)[i]) : ((const float*)w)[i];
}

__device__ __forceinline__ void report_error(int* err, int code, int d0, int d1, int d2) {
  if (err != nullptr && atomicCAS(err, 0, code) == 0) { err[1] = d0; err[2] = d1; err[3] = d2; }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the block; every thread gets the result.  The order depends only on blockDim.
__device__ __forceinline__ float block_sum(float v, float* smem32) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem32[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? smem32[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

static inline int launch_status() { return (int)cudaGetLastError(); }

// Streaming multiprocessors of the current device (asked once per device; 148 on a B200).
static inline int photon_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return 148; }
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) { cudaGetLastError(); n = 148; }
    cached[dev] = n;
  }
  return cached[dev];
}

// ---- programmatic dependent launch: a kernel may be scheduled while its predecessor in the stream drains.
// Everything it reads that the predecessor wrote must come after pdl_wait(); a kernel launched with
// launch_pdl must call pdl_wait() on every path, so that completion stays ordered along the stream.
// A kernel calls pdl_launch_dependents() once its main loop is done: earlier, the blocks of the next
// kernel would take the places of blocks of this grid that have not started yet.
// PHOTON_PDL=1: always on, PHOTON_PDL=0: off; unset: on for plain launches, off while the stream is
// being captured.  Measured on B200 at the Llama 3.2 1B shape: a prompt portion of 2,048 tokens (plain
// launches) gains 2 %; the decode step replayed as a CUDA graph takes 0.91 ms with it against 0.88 ms
// without.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool photon_pdl_enabled(cudaStream_t stream) {
  static int v = -1;                                 // 0 off, 1 on, 2 on outside capture
  if (v < 0) { const char* e = getenv("PHOTON_PDL"); v = (e == nullptr || e[0] == 0) ? 2 : (e[0] == '1' ? 1 : 0); }
  if (v != 2) return v == 1;
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) { cudaGetLastError(); return false; }
  return st == cudaStreamCaptureStatusNone;
}

template <typename... KArgs, typename... Args>
static inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = photon_pdl_enabled(stream) ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}
