"""The engine at real layer sizes against the plain implementation: the full Llama 3.2 1B shape in
float32 and bfloat16 (16 layers, vocabulary 128,256), and two layers of the 3B and 8B shapes (head size
128, three and four query heads per key/value head, intermediate 14,336, untied head)."""
import pytest
import torch

from helpers import TOL, plain_logits, random_ids, rel_err

pytestmark = pytest.mark.gpu

LLAMA3_SCALING = dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192)
SHAPES = {
    "1b": dict(hidden_size=2048, intermediate_size=8192, num_hidden_layers=16, num_attention_heads=32,
               num_key_value_heads=8, head_dim=64, vocab_size=128256, tie_word_embeddings=True),
    "3b_two_layers": dict(hidden_size=3072, intermediate_size=8192, num_hidden_layers=2, num_attention_heads=24,
                          num_key_value_heads=8, head_dim=128, vocab_size=32000, tie_word_embeddings=True),
    "8b_two_layers": dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=2, num_attention_heads=32,
                          num_key_value_heads=8, head_dim=128, vocab_size=32000, tie_word_embeddings=False),
}


@pytest.fixture(scope="module", params=list(SHAPES))
def model(request, tmp_path_factory):
    from photon_infer_b200.weights import write_random_model
    cfg = dict(architectures=["LlamaForCausalLM"], max_position_embeddings=131072, rms_norm_eps=1e-5,
               rope_theta=500000.0, rope_scaling=LLAMA3_SCALING, **SHAPES[request.param])
    folder = str(tmp_path_factory.mktemp(f"llama_{request.param}"))
    write_random_model(folder, cfg, seed=3, init_std=0.02, norm_std=0.0)
    return request.param, folder, cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_sizes_against_plain(model, dtype):
    from photon_infer_b200 import EngineOptions
    from photon_infer_b200.engine.loading import build_runner
    from photon_infer_b200.engine.runner import StepEntry
    name, folder, cfg = model
    ids = random_ids(170, cfg["vocab_size"], seed=11)
    want_rows = [0, 1, 63, 64, 127, 128, 149] + list(range(150, 170))
    want = plain_logits(folder, ids)[want_rows]
    runner = build_runner(folder, EngineOptions(dtype=dtype, block_size=16, max_cache_tokens=512, max_sequences=4))
    runner.cache.add_request("a")
    runner.cache.add_request("b")
    # a portion of 150 tokens (tcgen05 products and the many-rows attention in bfloat16), beside it another
    # request's portion; then 20 single tokens (weight-streaming products, split-key attention, CUDA graph)
    other = random_ids(40, cfg["vocab_size"], seed=12)
    res = runner.step([StepEntry("a", ids[:150], [0, 1, 63, 64, 127, 128, 149]), StepEntry("b", other, [])])
    got = [res.logits.cpu()]
    for t in ids[150:]:
        got.append(runner.step([StepEntry("a", [t], [0])]).logits.cpu())
    runner.check_device_errors()
    err = rel_err(torch.cat(got), want)
    assert err <= TOL[dtype], f"{name} {dtype}: {err:.3g}"
