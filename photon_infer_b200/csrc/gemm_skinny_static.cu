// The few-rows matrix product with its scratch in the library image: see gemm_skinny_static.h.
// The kernels and the launcher are those of gemm_skinny.cu, included here unchanged.
#include "gemm_skinny.cu"
#include "gemm_skinny_static.h"

// Tickets (int, one per row tile) in the first 32 KiB, partial sums (float) after them.  In host code
// this name is only a handle for cudaGetSymbolAddress, not a device address.
static __device__ __align__(256) unsigned char photon_static_scratch[PHOTON_STATIC_SCRATCH_BYTES];

#define PHOTON_STATIC_MAX_DEVICES 64
static unsigned char* g_scratch_of_device[PHOTON_STATIC_MAX_DEVICES];      // device addresses, one per GPU

PHOTON_API const char* photon_static_error_string(int code) {
  switch (code) {
    case 0: return "ok";
    case PHOTON_STATIC_TOO_LARGE:
      return "the product is larger than the static scratch allows: M <= 64 (32 with SwiGLU), N <= 131072";
    case PHOTON_ERR_UNSUPPORTED:
      return "K and the row strides of x and W (ldx, ldw) must be multiples of 8 elements, and x and W 16-byte aligned";
    case PHOTON_ERR_ARGUMENT: return "invalid argument";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error";
  }
}

PHOTON_API int photon_skinny_gemm_static(const void* x, long ldx, const void* W, long ldw, void* out, long ldo,
                                         int M, int N, int K, int epilogue, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || (epilogue == EPI_SWIGLU && M > 32) || N > PHOTON_STATIC_MAX_ROWS) return PHOTON_STATIC_TOO_LARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= PHOTON_STATIC_MAX_DEVICES) return PHOTON_ERR_ARGUMENT;
  // two threads that make the first call together both look the address up and store the same value
  unsigned char* base = __atomic_load_n(&g_scratch_of_device[dev], __ATOMIC_ACQUIRE);
  if (base == nullptr) {
    // first call on this device: the symbol's address on the current device
    e = cudaGetSymbolAddress((void**)&base, photon_static_scratch);
    if (e != cudaSuccess) return (int)e;
    __atomic_store_n(&g_scratch_of_device[dev], base, __ATOMIC_RELEASE);
  }
  int* tickets = reinterpret_cast<int*>(base);
  float* shares = reinterpret_cast<float*>(base + 32768);
  const int num_tickets = 32768 / (int)sizeof(int);
  // the tickets must be zero when the kernel starts, whatever an earlier call left
  e = cudaMemsetAsync(tickets, 0, 32768, stream);
  if (e != cudaSuccess) return (int)e;
  return photon_skinny_gemm(x, ldx, W, ldw, out, ldo, M, N, K, epilogue, shares, (long)PHOTON_STATIC_SHARE_FLOATS,
                            tickets, num_tickets, stream);
}
