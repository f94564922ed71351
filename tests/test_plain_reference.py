"""The plain implementation against logits made by the reference's own CPU kernels."""
import json
import os

import numpy as np
import torch

from plain.llama_plain import PlainLlama, argmax_first, inverse_cdf_sample, temperature_probabilities

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_tiny.npz")


def _load():
    z = np.load(GOLDEN)
    config = json.loads(bytes(z["config"]).decode())
    weights = {k: torch.from_numpy(z[k]) for k in z.files if k not in ("ids", "logits", "config")}
    return config, weights, z["ids"].tolist(), torch.from_numpy(z["logits"])


def test_plain_matches_reference_kernels_fp32():
    config, weights, ids, golden = _load()
    got = PlainLlama(config, weights, dtype=torch.float32).logits(ids)
    assert got.shape == golden.shape
    # both sides are 32-bit with different summation orders
    assert float((got - golden).abs().max()) <= 2e-6 * float(golden.abs().max()) + 1e-6


def test_plain_fp64_close_to_reference_kernels():
    config, weights, ids, golden = _load()
    got = PlainLlama(config, weights, dtype=torch.float64).logits(ids)
    assert float((got - golden).abs().max()) <= 2e-6 * float(golden.abs().max()) + 1e-6


def test_prefix_independence():
    """Causality: logits of a prefix do not change when tokens follow."""
    config, weights, ids, _ = _load()
    m = PlainLlama(config, weights)
    full = m.logits(ids)
    part = m.logits(ids[:9])
    assert float((full[:9] - part).abs().max()) < 1e-6


def test_half_split_equals_interleaved_after_permutation():
    """The two pair conventions differ only by a permutation of q/k rows."""
    config, weights, ids, golden = _load()
    hd = config["hidden_size"] // config["num_attention_heads"]
    perm_head = torch.cat([torch.arange(0, hd, 2), torch.arange(1, hd, 2)])
    w2 = dict(weights)
    for l in range(config["num_hidden_layers"]):
        for name, heads in (("q_proj", config["num_attention_heads"]), ("k_proj", config["num_key_value_heads"])):
            key = f"model.layers.{l}.self_attn.{name}.weight"
            w = weights[key].view(heads, hd, -1)
            w2[key] = w[:, perm_head, :].reshape(heads * hd, -1).contiguous()
    cfg2 = dict(config, rope_interleaved=False)
    got = PlainLlama(cfg2, w2).logits(ids)
    assert float((got - golden).abs().max()) <= 2e-6 * float(golden.abs().max()) + 1e-6


def test_window_limits_keys():
    from plain.llama_plain import causal_attention
    torch.manual_seed(0)
    q, k, v = torch.randn(10, 2, 8), torch.randn(10, 1, 8), torch.randn(10, 1, 8)
    full = causal_attention(q, k, v)
    win = causal_attention(q, k, v, window=3)
    assert torch.allclose(full[:3], win[:3], atol=1e-6)
    # position 9 with window 3 sees keys 7, 8, 9 only
    alone = causal_attention(q[7:], k[7:], v[7:])
    assert torch.allclose(win[9], alone[2], atol=1e-6)
    assert not torch.allclose(full[9], win[9], atol=1e-4)


def test_sampling_helpers():
    l = torch.tensor([0.5, 2.0, 2.0, -1.0])
    assert argmax_first(l) == 1
    p = temperature_probabilities(l, 0.8)
    assert abs(float(p.sum()) - 1.0) < 1e-6
    assert inverse_cdf_sample(p, 0.0) == 0
    assert inverse_cdf_sample(p, float(p[0]) + 1e-4) == 1
    assert inverse_cdf_sample(p, 1.0) in (2, 3)
