// Decode throughput of lumia431/photon_infer itself, through its own public API and stock batched path,
// at the Llama 3.2 1B shape with random weights.  Nothing of photon_infer_b200 is on this path.
//
// The calls are those of the reference's own batched demo (demo/batched_infer_multi_prompts.cpp:82-227):
// LLaMAModel(config) -> set_* weights (what CheckpointLoader::load_weights does,
// src/io/checkpoint.cpp:131-314) -> init() -> quantize_weights(128) (its only matrix-product path on CUDA,
// src/ops/matmul.cpp:169-172) -> init_paged_cache(num_blocks, 16) -> allocate_sequence per request ->
// forward_batched(tokens, positions, seq_ids, logits) once per position with all requests in lock step
// (prompts first, then decode steps) -> argmax_sampling_launch -> cudaMemcpy of the ids to the host.
// Weights are N(0, 0.02) and norm weights 1, seeded, as its model test draws them
// (tests/model/test_llama_model.cpp:31-42); token ids are seeded uniform numbers.
//
// Prints ONE JSON line: decoded tokens per second over --steps decode steps after --warmup untimed ones,
// timed with CUDA events ("value") and with the host clock around the same loop ("e2e": the loop already
// copies ids to the device and sampled ids back in every step, because the reference's API takes host vectors).
#include <cuda_runtime.h>

#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "photon/arch/llama_model.hpp"
#include "photon/ops/kernels/cuda/sampling_kernel.cuh"
#include "photon/runtime/kv_cache_manager.hpp"

using namespace photon;
using namespace photon::model;

namespace {

struct Rng {                                   // xorshift128+, one stream per (seed, tensor, thread)
  uint64_t a, b;
  explicit Rng(uint64_t seed) : a(seed * 0x9E3779B97F4A7C15ull + 1), b(seed ^ 0xD1B54A32D192ED03ull) {
    for (int i = 0; i < 8; ++i) next();
  }
  uint64_t next() {
    uint64_t x = a, y = b;
    a = y;
    x ^= x << 23;
    b = x ^ y ^ (x >> 17) ^ (y >> 26);
    return b + y;
  }
  double uniform() { return (static_cast<double>(next() >> 11) + 0.5) * (1.0 / 9007199254740992.0); }
};

void fill_normal(float* p, size_t n, float std_dev, uint64_t seed) {
  const unsigned threads = std::max(1u, std::min(16u, std::thread::hardware_concurrency()));
  std::vector<std::thread> pool;
  for (unsigned t = 0; t < threads; ++t) {
    pool.emplace_back([=]() {
      Rng rng(seed * 1315423911ull + t);
      const size_t lo = n * t / threads, hi = n * (t + 1) / threads;
      for (size_t i = lo; i < hi; i += 2) {    // Box-Muller, two values per draw
        const double r = std::sqrt(-2.0 * std::log(rng.uniform())), phi = 6.283185307179586 * rng.uniform();
        p[i] = static_cast<float>(r * std::cos(phi)) * std_dev;
        if (i + 1 < hi) p[i + 1] = static_cast<float>(r * std::sin(phi)) * std_dev;
      }
    });
  }
  for (auto& th : pool) th.join();
}

Tensor make(std::vector<i32> dims, float std_dev, uint64_t seed) {
  auto r = Tensor::create(dims, DataType::Float32, DeviceType::CPU);
  if (!r) { std::fprintf(stderr, "tensor: %s\n", r.error().message().c_str()); std::exit(3); }
  Tensor t = std::move(r.value());
  if (std_dev > 0.f) fill_normal(t.ptr<f32>(), t.size(), std_dev, seed);
  else for (usize i = 0; i < t.size(); ++i) t.ptr<f32>()[i] = 1.0f;
  return t;
}

#define MUST(expr)                                                                          \
  do {                                                                                      \
    auto must_result = (expr);                                                              \
    if (!must_result) {                                                                     \
      std::fprintf(stderr, "%s: %s\n", #expr, must_result.error().message().c_str());       \
      std::printf("{\"impl\": \"reference\", \"unavailable\": \"the reference returned an error from %s\"}\n", #expr); \
      return 0;                                                                             \
    }                                                                                       \
  } while (0)

int arg(int argc, char** argv, const char* name, int fallback) {
  for (int i = 1; i + 1 < argc; ++i)
    if (std::strcmp(argv[i], name) == 0) return std::atoi(argv[i + 1]);
  return fallback;
}

}  // namespace

int main(int argc, char** argv) {
  const int batch = arg(argc, argv, "--batch", 8), prompt_len = arg(argc, argv, "--prompt", 512);
  const int steps = arg(argc, argv, "--steps", 20), warmup = arg(argc, argv, "--warmup", 5);
  const int layers = arg(argc, argv, "--layers", 16), generated = arg(argc, argv, "--generated", 256);
  const uint64_t seed = static_cast<uint64_t>(arg(argc, argv, "--seed", 0));

  TransformerConfig config;
  config.dim = 2048;
  config.hidden_dim = 8192;
  config.n_layers = layers;
  config.n_heads = 32;
  config.n_kv_heads = 8;
  config.vocab_size = 128256;
  config.seq_len = 4096;                         // the longest context its paged kernels take
  config.head_size = config.dim / config.n_heads;
  config.norm_eps = 1e-5f;
  config.device = DeviceType::CUDA;
  config.compute_derived();
  const i32 D = config.dim, KV = config.kv_dim, I = config.hidden_dim, V = config.vocab_size;

  std::fprintf(stderr, "[reference] drawing weights ...\n");
  LLaMAModel model(config);
  MUST(model.set_embedding(make({V, D}, 0.02f, seed * 1000 + 1)));
  MUST(model.set_final_norm(make({D}, 0.f, 0)));
  for (i32 l = 0; l < layers; ++l) {
    auto& b = model.get_block(l);
    const uint64_t s = seed * 1000 + 10 + static_cast<uint64_t>(l) * 16;
    MUST(b.set_attn_norm(make({D}, 0.f, 0)));
    MUST(b.set_wq(make({D, D}, 0.02f, s + 1)));
    MUST(b.set_wk(make({KV, D}, 0.02f, s + 2)));
    MUST(b.set_wv(make({KV, D}, 0.02f, s + 3)));
    MUST(b.set_wo(make({D, D}, 0.02f, s + 4)));
    MUST(b.set_ffn_norm(make({D}, 0.f, 0)));
    MUST(b.set_w1(make({I, D}, 0.02f, s + 5)));
    MUST(b.set_w2(make({D, I}, 0.02f, s + 6)));
    MUST(b.set_w3(make({I, D}, 0.02f, s + 7)));
  }
  // tied head: the loader hands the classifier a copy of the embedding (src/io/checkpoint.cpp:305-313)
  MUST(model.set_classifier(make({V, D}, 0.02f, seed * 1000 + 1)));
  MUST(model.init());
  std::fprintf(stderr, "[reference] quantizing (its only CUDA product path) ...\n");
  MUST(model.quantize_weights(128));
  const i32 block_size = 16;
  const i32 per_seq = prompt_len + generated + 10;
  const i32 num_blocks = batch * ((per_seq + block_size - 1) / block_size + 1);
  MUST(model.init_paged_cache(num_blocks, block_size));
  auto* cache = model.paged_cache_manager();
  std::vector<i32> seq_ids(batch);
  for (i32 i = 0; i < batch; ++i) {
    seq_ids[i] = i;
    MUST(cache->allocate_sequence(i, per_seq));
  }
  auto logits_r = Tensor::create({batch, V}, DataType::Float32, DeviceType::CUDA);
  if (!logits_r) {
    std::printf("{\"impl\": \"reference\", \"unavailable\": \"the reference could not allocate its logits\"}\n");
    return 0;
  }
  Tensor logits = std::move(logits_r.value());

  Rng ids(seed + 77);
  std::vector<i32> tokens(batch), positions(batch), sampled(batch);
  std::fprintf(stderr, "[reference] %d prompt positions in lock step ...\n", prompt_len);
  for (i32 pos = 0; pos < prompt_len; ++pos) {
    for (i32 i = 0; i < batch; ++i) { tokens[i] = static_cast<i32>(ids.next() % static_cast<uint64_t>(V)); positions[i] = pos; }
    MUST(model.forward_batched(tokens, positions, seq_ids, logits));
  }
  i32* sampled_gpu = nullptr;
  if (cudaMalloc(&sampled_gpu, batch * sizeof(i32)) != cudaSuccess) return 4;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  double wall = 0.0;
  for (i32 step = 0; step < warmup + steps; ++step) {
    if (step == warmup) {
      cudaDeviceSynchronize();
      cudaEventRecord(e0);
      wall = std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
    }
    for (i32 i = 0; i < batch; ++i) {
      tokens[i] = step == 0 ? static_cast<i32>(ids.next() % static_cast<uint64_t>(V)) : sampled[i];
      positions[i] = prompt_len + step;
    }
    MUST(model.forward_batched(tokens, positions, seq_ids, logits));
    MUST(photon::kernels::cuda::argmax_sampling_launch(logits.ptr<f32>(), sampled_gpu, batch, V, nullptr));
    cudaMemcpy(sampled.data(), sampled_gpu, batch * sizeof(i32), cudaMemcpyDeviceToHost);
  }
  cudaEventRecord(e1);
  cudaDeviceSynchronize();
  wall = std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count() - wall;
  float ms = 0.f;
  cudaEventElapsedTime(&ms, e0, e1);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    std::printf("{\"impl\": \"reference\", \"unavailable\": \"CUDA error in the reference's path: %s\"}\n", cudaGetErrorString(err));
    return 0;
  }
  const i32 max_blocks = cache->get_max_blocks_per_seq();
  // per step: ids, positions, request ids once; in every layer the block table and the lengths again
  const long h2d = 3L * batch * 4 + static_cast<long>(layers) * (static_cast<long>(batch) * max_blocks * 4 + batch * 4);
  std::printf(
      "{\"metric\": \"decode tokens/s, Llama 3.2 1B shape, batch %d\", \"value\": %.1f, \"unit\": \"tokens/s\", "
      "\"n_gpus\": 1, \"steps\": %d, \"warmup\": %d, \"ms_per_step\": %.4f, \"higher_is_better\": true, "
      "\"scaling\": \"weak\", \"dtype\": \"fp32 products on weights it quantizes to int8 and dequantizes once (its only CUDA path)\", "
      "\"data\": \"synthetic token ids, random weights N(0, 0.02)\", \"impl\": \"reference\", "
      "\"config\": {\"model\": \"llama-3.2-1b-shape\", \"layers\": %d, \"layers_of_model\": 16, \"hidden\": 2048, \"q_heads\": 32, "
      "\"kv_heads\": 8, \"head_dim\": 64, \"intermediate\": 8192, \"vocab\": 128256, \"global_batch\": %d, \"seq_len\": 4096, "
      "\"prompt_len\": %d, \"generated\": %d, \"page_size\": 16, \"parallelism\": \"single\"}, "
      "\"e2e\": {\"value\": %.1f, \"unit\": \"tokens/s\", \"h2d_bytes_per_step\": %ld, \"d2h_bytes_per_step\": %d}}\n",
      batch, batch * steps / (ms / 1e3), steps, warmup, ms / steps, layers, batch, prompt_len, generated,
      batch * steps / wall, h2d, batch * 4);
  cudaFree(sampled_gpu);
  return 0;
}
