"""A long request: 6,144 tokens fed in portions of 2,048, then single tokens, against the plain
implementation.  The block table of the request spans hundreds of pages, the decode steps split
their keys over many blocks, and the portions start deep inside the request."""
import pytest
import torch

from helpers import TOL, plain_logits, random_ids, rel_err

pytestmark = pytest.mark.gpu

CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=128, intermediate_size=256, num_hidden_layers=2,
           num_attention_heads=8, num_key_value_heads=2, head_dim=64, vocab_size=512,
           max_position_embeddings=16384, rms_norm_eps=1e-5, rope_theta=500000.0,
           rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                             original_max_position_embeddings=2048),
           tie_word_embeddings=True)


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    from photon_infer_b200.weights import write_random_model
    f = str(tmp_path_factory.mktemp("long_context"))
    write_random_model(f, CFG, seed=9, init_std=0.05, norm_std=0.1)
    return f


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_request_in_portions_then_single_tokens(folder, dtype):
    from photon_infer_b200 import EngineOptions
    from photon_infer_b200.engine.loading import build_runner
    from photon_infer_b200.engine.runner import StepEntry
    n, tail = 6144, 12
    ids = random_ids(n + tail, CFG["vocab_size"], seed=4)
    runner = build_runner(folder, EngineOptions(dtype=dtype, block_size=16, max_cache_tokens=n + 64, max_sequences=2))
    runner.cache.add_request("x")
    got, rows = [], []
    for lo in range(0, n, 2048):
        want = [0, 1, 1023, 2046, 2047]
        got.append(runner.step([StepEntry("x", ids[lo:lo + 2048], want)]).logits.cpu())
        rows += [lo + w for w in want]
    for p in range(n, n + tail):
        got.append(runner.step([StepEntry("x", [ids[p]], [0])]).logits.cpu())
        rows.append(p)
    runner.check_device_errors()
    want_logits = plain_logits(folder, ids)[rows]
    assert rel_err(torch.cat(got), want_logits) <= TOL[dtype]
