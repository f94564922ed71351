// Row-wise kernels of the decoder: embedding lookup, residual add fused with RMSNorm
// (on all rows or on a list of rows), SwiGLU.  All arithmetic is 32-bit; storage is
// float or bfloat16.  Formulas: include/photon/ops/kernels/rmsnorm_kernel.hpp:71-86
// (w * (x * 1/sqrt(mean(x^2)+eps))), include/photon/ops/kernels/swiglu_kernel.hpp:67-76
// (g / (1 + exp(-g)) * u), include/photon/ops/kernels/embedding_kernel.hpp:85-121.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embedding_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                 float* __restrict__ out, int H, int V, int* err) {
  const int t = blockIdx.x;
  const int id = ids[t];
  float* o = out + (size_t)t * H;
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) report_error(err, PHOTON_DEV_BAD_TOKEN, t, id, V);
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const TW* row = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(row[i]);
}

PHOTON_API int photon_embedding(const int* ids, const void* table, int table_dtype, float* out,
                                int T, int H, int V, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == PHOTON_BF16)
    embedding_kernel<bf16><<<T, threads, 0, stream>>>(ids, (const bf16*)table, out, H, V, err);
  else
    embedding_kernel<float><<<T, threads, 0, stream>>>(ids, (const float*)table, out, H, V, err);
  return launch_status();
}

// ---------------------------------------------------------------- add + RMSNorm
// residual (float, in place) += delta; out = w * (residual * r).  rows == nullptr: row = blockIdx.x
// of both residual and out.  rows != nullptr: reads row rows[blockIdx.x] and does NOT write the sum
// back (the listed rows are only read; out has one row per list entry).
template <typename T> struct Quad;            // four consecutive elements as one load or store
template <> struct Quad<float> {
  __device__ static void load(const float* p, float* f) { const float4 r = *reinterpret_cast<const float4*>(p); f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w; }
  __device__ static void store(float* p, const float* f) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Quad<bf16> {
  __device__ static void load(const bf16* p, float* f) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  }
  __device__ static void store(bf16* p, const float* f) {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    uint2 r;
    r.x = *reinterpret_cast<uint32_t*>(&a);
    r.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
  }
};

// VEC: rows are read and written four elements at a time (H a multiple of 4, aligned pointers).
template <typename TD, typename TO, bool VEC>
__global__ void add_rmsnorm_kernel(const TD* delta, float* residual,          // written by earlier kernels that may
                                   const void* __restrict__ w, int w_bf16,    // still run when this one starts: no
                                   TO* out, const int* rows, int H, float eps) {  // read-only path for them
  __shared__ float red[32];
  extern __shared__ __align__(16) float stash[];               // H floats: the summed row
  pdl_wait();
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* res = residual + (size_t)r * H;
  const TD* d = delta ? delta + (size_t)r * H : nullptr;
  float ss = 0.f;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float v[4], dv[4];
      Quad<float>::load(res + i, v);
      if (d) {
        Quad<TD>::load(d + i, dv);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] += dv[e];
      }
      Quad<float>::store(stash + i, v);
#pragma unroll
      for (int e = 0; e < 4; ++e) ss += v[e] * v[e];
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = res[i];
      if (d) v += to_f32(d[i]);
      stash[i] = v;
      ss += v * v;
    }
  }
  ss = block_sum(ss, red);
  pdl_launch_dependents();                         // the next kernel may be scheduled while the row is written
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  TO* o = out + (size_t)blockIdx.x * H;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float v[4], wv[4], y[4];
      Quad<float>::load(stash + i, v);
      if (w_bf16) Quad<bf16>::load((const bf16*)w + i, wv); else Quad<float>::load((const float*)w + i, wv);
      if (d && !rows) Quad<float>::store(res + i, v);
#pragma unroll
      for (int e = 0; e < 4; ++e) y[e] = wv[e] * (v[e] * inv);
      Quad<TO>::store(o + i, y);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = stash[i];
      if (d && !rows) res[i] = v;
      o[i] = from_f32<TO>(load_w(w, w_bf16, i) * (v * inv));
    }
  }
}

template <typename TD, typename TO>
static int add_rmsnorm_launch(const void* delta, float* residual, const void* w, int w_bf16, void* out,
                              const int* rows, int n, int H, float eps, cudaStream_t stream) {
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return PHOTON_ERR_UNSUPPORTED;
  const bool vec = (H % 4 == 0) && ((uintptr_t)delta % 16 == 0) && ((uintptr_t)residual % 16 == 0) &&
                   ((uintptr_t)w % 16 == 0) && ((uintptr_t)out % 16 == 0);
  if (smem > 48 * 1024) {
    cudaError_t e = vec ? cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO, true>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                        : cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO, false>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  int threads = 128;
  while (threads < 1024 && threads * 4 < H) threads <<= 1;   // depends on H only
  if (vec)
    return launch_pdl(add_rmsnorm_kernel<TD, TO, true>, dim3(n), dim3(threads), smem, stream, (const TD*)delta,
                      residual, w, w_bf16, (TO*)out, rows, H, eps);
  return launch_pdl(add_rmsnorm_kernel<TD, TO, false>, dim3(n), dim3(threads), smem, stream, (const TD*)delta,
                    residual, w, w_bf16, (TO*)out, rows, H, eps);
}

// delta may be null (plain norm).  delta_dtype / out_dtype: PHOTON_F32 or PHOTON_BF16.
PHOTON_API int photon_add_rmsnorm(const void* delta, int delta_dtype, float* residual, const void* w,
                                  int w_dtype, void* out, int out_dtype, const int* rows, int n, int H,
                                  float eps, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int wb = (w_dtype == PHOTON_BF16);
  if (delta_dtype == PHOTON_BF16 && out_dtype == PHOTON_BF16)
    return add_rmsnorm_launch<bf16, bf16>(delta, residual, w, wb, out, rows, n, H, eps, stream);
  if (delta_dtype == PHOTON_F32 && out_dtype == PHOTON_F32)
    return add_rmsnorm_launch<float, float>(delta, residual, w, wb, out, rows, n, H, eps, stream);
  if (delta_dtype == PHOTON_F32 && out_dtype == PHOTON_BF16)
    return add_rmsnorm_launch<float, bf16>(delta, residual, w, wb, out, rows, n, H, eps, stream);
  if (delta_dtype == PHOTON_BF16 && out_dtype == PHOTON_F32)
    return add_rmsnorm_launch<bf16, float>(delta, residual, w, wb, out, rows, n, H, eps, stream);
  return PHOTON_ERR_ARGUMENT;
}

// ---------------------------------------------------------------- SwiGLU
// gate_up [T, 2*I]: columns [0, I) are the gate, [I, 2I) the up projection.  out [T, I].
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int I, size_t total) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_f32(gate_up[t * 2 * I + i]);
    const float u = to_f32(gate_up[t * 2 * I + I + i]);
    const float s = g / (1.0f + expf(-g));
    out[idx] = from_f32<T>(s * u);
  }
}

// The same, 16 bytes per load: I a multiple of the elements in 16 bytes, aligned pointers.
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int I, size_t total_vecs) {
  constexpr int N = 16 / sizeof(T);
  const int per_row = I / N;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total_vecs; idx += stride) {
    const size_t t = idx / per_row;
    const int i = (int)(idx - t * per_row) * N;
    const uint4 gv = *reinterpret_cast<const uint4*>(gate_up + t * 2 * I + i);
    const uint4 uv = *reinterpret_cast<const uint4*>(gate_up + t * 2 * I + I + i);
    const T* gp = reinterpret_cast<const T*>(&gv);
    const T* up = reinterpret_cast<const T*>(&uv);
    uint4 ov;
    T* op = reinterpret_cast<T*>(&ov);
#pragma unroll
    for (int e = 0; e < N; ++e) {
      const float g = to_f32(gp[e]);
      op[e] = from_f32<T>(g / (1.0f + expf(-g)) * to_f32(up[e]));
    }
    *reinterpret_cast<uint4*>(out + t * I + i) = ov;
  }
}

PHOTON_API int photon_swiglu(const void* gate_up, void* out, int dtype, int T, int I, cudaStream_t stream) {
  const size_t total = (size_t)T * I;
  if (total == 0) return 0;
  const int threads = 256;
  const int n = dtype == PHOTON_BF16 ? 8 : 4;
  const bool vec = (I % n == 0) && ((uintptr_t)gate_up % 16 == 0) && ((uintptr_t)out % 16 == 0);
  const size_t work = vec ? total / n : total;
  size_t blocks = (work + threads - 1) / threads;
  const size_t cap = (size_t)photon_sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (dtype == PHOTON_BF16) {
    if (vec) swiglu_vec_kernel<bf16><<<(int)blocks, threads, 0, stream>>>((const bf16*)gate_up, (bf16*)out, I, work);
    else swiglu_kernel<bf16><<<(int)blocks, threads, 0, stream>>>((const bf16*)gate_up, (bf16*)out, I, total);
  } else {
    if (vec) swiglu_vec_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, I, work);
    else swiglu_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, I, total);
  }
  return launch_status();
}
