#!/usr/bin/env python3
"""Makes ``tests/golden/reference_tiny.npz``: logits of a tiny random Llama decoder
computed by lumia431/photon_infer's own CPU kernels.

The reference's whole-model CPU path cannot run here (its blocks are built on Eigen,
which is not installed), but its naive kernels are header-only templates.  This
script writes a small C++ harness that includes those headers BY PATH from a
checkout of the reference (nothing of it is copied into this repository), chains the
kernels token by token in the order of src/arch/transformer_block.cpp:199-296 and
src/arch/llama_model.cpp:186-272, and dumps the logits of every position.

    python tests/golden/make_golden.py --reference /path/to/photon_infer

The model matches the constants that the reference fixes in code: rope base 10000,
no frequency scaling, neighbouring pairs, eps 1e-5, head_dim = hidden / heads.
The weights (seeded) and the token ids are stored beside the logits, so the test
needs neither the reference nor this script.
"""
import argparse
import json
import os
import subprocess
import tempfile

import numpy as np

CFG = dict(vocab=64, hidden=32, inter=48, layers=2, heads=4, kv_heads=2, seq=24)

HARNESS = r"""
#include <cstdio>
#include <cstring>
#include <vector>
#include <span>
#include "photon/ops/kernels/rmsnorm_kernel.hpp"
#include "photon/ops/kernels/matmul_kernel.hpp"
#include "photon/ops/kernels/rope_kernel.hpp"
#include "photon/ops/kernels/mha_kernel.hpp"
#include "photon/ops/kernels/swiglu_kernel.hpp"
#include "photon/ops/kernels/add_kernel.hpp"
using namespace photon;
using namespace photon::kernels;
static std::vector<float> rd(FILE* f, size_t n) { std::vector<float> v(n); if (fread(v.data(), 4, n, f) != n) { perror("short read"); exit(2);} return v; }
int main(int argc, char** argv) {
  int V=%(vocab)d, H=%(hidden)d, I=%(inter)d, L=%(layers)d, NH=%(heads)d, NKV=%(kv_heads)d, S=%(seq)d;
  int HS = H / NH, KV = NKV * HS, MUL = NH / NKV;
  FILE* f = fopen(argv[1], "rb");
  std::vector<int> ids(S); if (fread(ids.data(), 4, S, f) != (size_t)S) return 2;
  auto emb = rd(f, (size_t)V*H);
  std::vector<std::vector<float>> an(L), wq(L), wk(L), wv(L), wo(L), fn(L), w1(L), w2(L), w3(L);
  for (int l = 0; l < L; ++l) { an[l]=rd(f,H); wq[l]=rd(f,(size_t)H*H); wk[l]=rd(f,(size_t)KV*H); wv[l]=rd(f,(size_t)KV*H);
    wo[l]=rd(f,(size_t)H*H); fn[l]=rd(f,H); w1[l]=rd(f,(size_t)I*H); w3[l]=rd(f,(size_t)I*H); w2[l]=rd(f,(size_t)H*I); }
  auto fin = rd(f, H); fclose(f);
  std::vector<float> sinc((size_t)S*HS), cosc((size_t)S*HS);
  compute_rope_cache<float>(sinc, cosc, S, HS);
  std::vector<std::vector<float>> K(L, std::vector<float>((size_t)S*KV)), Vc(L, std::vector<float>((size_t)S*KV));
  std::vector<float> x(H), h(H), q(H), k(KV), v(KV), a(H), o(H), g(I), u(I), s(I), d(H), score((size_t)NH*S), logits(V);
  FILE* out = fopen(argv[2], "wb");
  for (int pos = 0; pos < S; ++pos) {
    std::memcpy(x.data(), emb.data() + (size_t)ids[pos]*H, H*4);          // embedding: row copy
    for (int l = 0; l < L; ++l) {
      rmsnorm_naive<float>(x, an[l], h, H, 1e-5f);
      matmul_gemv_naive<float>(h, wq[l], q, H, H);
      matmul_gemv_naive<float>(h, wk[l], k, KV, H);
      matmul_gemv_naive<float>(h, wv[l], v, KV, H);
      rope_naive<float>(q, k, sinc, cosc, pos, H, KV, HS);
      std::memcpy(K[l].data() + (size_t)pos*KV, k.data(), KV*4);
      std::memcpy(Vc[l].data() + (size_t)pos*KV, v.data(), KV*4);
      mha_naive<float>(q, K[l], Vc[l], a, score, pos, KV, NH, HS, S, MUL);
      matmul_gemv_naive<float>(a, wo[l], o, H, H);
      add_naive<float>(x, o, x, H);
      rmsnorm_naive<float>(x, fn[l], h, H, 1e-5f);
      matmul_gemv_naive<float>(h, w1[l], g, I, H);
      matmul_gemv_naive<float>(h, w3[l], u, I, H);
      swiglu_naive<float>(g, u, s, I);
      matmul_gemv_naive<float>(s, w2[l], d, H, I);
      add_naive<float>(x, d, x, H);
    }
    rmsnorm_naive<float>(x, fin, h, H, 1e-5f);
    matmul_gemv_naive<float>(h, emb, logits, V, H);                       // tied output head
    fwrite(logits.data(), 4, V, out);
  }
  fclose(out);
  return 0;
}
"""


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="a checkout of lumia431/photon_infer (its include/ folder is compiled against)")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(__file__), "reference_tiny.npz"))
    args = ap.parse_args()
    c = CFG
    hs = c["hidden"] // c["heads"]
    kv = c["kv_heads"] * hs
    rng = np.random.default_rng(20240)
    ids = rng.integers(0, c["vocab"], size=c["seq"]).astype(np.int32)

    def w(*shape, std=0.08):
        return (rng.standard_normal(shape) * std).astype(np.float32)

    def norm_w():
        return (1.0 + 0.1 * rng.standard_normal(c["hidden"])).astype(np.float32)

    tensors = {"model.embed_tokens.weight": w(c["vocab"], c["hidden"])}
    order = [tensors["model.embed_tokens.weight"]]
    for l in range(c["layers"]):
        p = f"model.layers.{l}."
        layer = {
            p + "input_layernorm.weight": norm_w(),
            p + "self_attn.q_proj.weight": w(c["hidden"], c["hidden"]),
            p + "self_attn.k_proj.weight": w(kv, c["hidden"]),
            p + "self_attn.v_proj.weight": w(kv, c["hidden"]),
            p + "self_attn.o_proj.weight": w(c["hidden"], c["hidden"]),
            p + "post_attention_layernorm.weight": norm_w(),
            p + "mlp.gate_proj.weight": w(c["inter"], c["hidden"]),
            p + "mlp.up_proj.weight": w(c["inter"], c["hidden"]),
            p + "mlp.down_proj.weight": w(c["hidden"], c["inter"]),
        }
        tensors.update(layer)
        order.extend(layer.values())
    tensors["model.norm.weight"] = norm_w()
    order.append(tensors["model.norm.weight"])

    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "harness.cpp")
        with open(src, "w") as f:
            f.write(HARNESS % c)
        exe = os.path.join(tmp, "harness")
        subprocess.check_call(["g++", "-std=c++20", "-O1", "-ffp-contract=off",
                               "-I", os.path.join(args.reference, "include"), src, "-o", exe])
        blob = os.path.join(tmp, "in.bin")
        with open(blob, "wb") as f:
            f.write(ids.tobytes())
            for t in order:
                f.write(np.ascontiguousarray(t).tobytes())
        res = os.path.join(tmp, "out.bin")
        subprocess.check_call([exe, blob, res])
        logits = np.fromfile(res, dtype=np.float32).reshape(c["seq"], c["vocab"])

    config = {
        "architectures": ["LlamaForCausalLM"], "hidden_size": c["hidden"],
        "intermediate_size": c["inter"], "num_hidden_layers": c["layers"],
        "num_attention_heads": c["heads"], "num_key_value_heads": c["kv_heads"],
        "vocab_size": c["vocab"], "max_position_embeddings": c["seq"], "rms_norm_eps": 1e-5,
        "rope_theta": 10000.0, "rope_interleaved": True, "tie_word_embeddings": True,
    }
    np.savez_compressed(args.out, ids=ids, logits=logits,
                        config=np.frombuffer(json.dumps(config).encode(), dtype=np.uint8), **tensors)
    print("wrote", args.out, logits.shape, float(np.abs(logits).max()))


if __name__ == "__main__":
    main()
