"""The llama3 frequency-scaling rule, pinned from outside the two implementations.

lumia431/photon_infer has no frequency scaling (its rotation base is fixed,
include/photon/ops/kernels/rope_kernel.hpp:68-74), so the logits made by its kernels under
``tests/golden/`` cannot anchor this rule.  The product (``parts/rope.py``) and the plain
implementation (``tests/plain/llama_plain.py``) both state it in wavelengths.  This file states it a
third way, in turns: a frequency ``f`` makes ``n = orig * f / (2 pi)`` full turns over the original
context; fewer than ``low`` turns: ``f / factor``; more than ``high``: unchanged; between them the two
are blended with weight ``s = (n - low) / (high - low)`` on the unchanged one.  It also pins numbers:
the frequencies inside the blended band for the Llama 3.2 1B and Llama 3.1 8B parameters were worked
out once in float64 from that statement and are written here as literals, so that a change of either
implementation shows up as a changed number and not as two implementations drifting together.
"""
import math

import pytest
import torch

from plain.llama_plain import rope_inverse_frequencies
from photon_infer_b200.parts.rope import inverse_frequencies

LLAMA3 = {
    "1b": (64, 5e5, dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                         original_max_position_embeddings=8192)),
    "8b": (128, 5e5, dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=8192)),
    "tiny_b": (32, 5e5, dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                             original_max_position_embeddings=64)),
}
# index of the frequency -> value, for every frequency that falls inside the blended band
BAND = {
    "1b": {15: 0.0012905478943139315, 16: 0.00042955679236911237, 17: 9.708287689136341e-05},
    "8b": {29: 0.0021665708627551794, 30: 0.0013718935661017895, 31: 0.0008567514014430344,
           32: 0.000524846138432622, 33: 0.00031269373721443117, 34: 0.00017850780568551272},
    "tiny_b": {2: 0.07940300554037094},
}


def _in_turns(head_dim, theta, s):
    out = []
    for j in range(head_dim // 2):
        f = theta ** (-(2 * j) / head_dim)
        n = s["original_max_position_embeddings"] * f / (2 * math.pi)
        if n < s["low_freq_factor"]:
            f = f / s["factor"]
        elif n <= s["high_freq_factor"]:
            w = (n - s["low_freq_factor"]) / (s["high_freq_factor"] - s["low_freq_factor"])
            f = f * (w + (1 - w) / s["factor"])
        out.append(f)
    return out


@pytest.mark.parametrize("name", list(LLAMA3))
def test_both_implementations_follow_the_rule_stated_in_turns(name):
    d, theta, s = LLAMA3[name]
    want = torch.tensor(_in_turns(d, theta, s), dtype=torch.float64)
    for got in (rope_inverse_frequencies(d, theta, s), inverse_frequencies(d, theta, s)):
        assert got.dtype == torch.float32 and got.shape == (d // 2,)
        assert float(((got.double() - want) / want).abs().max()) < 1e-7      # one float32 rounding


@pytest.mark.parametrize("name", list(LLAMA3))
def test_pinned_numbers_and_shape_of_the_curve(name):
    d, theta, s = LLAMA3[name]
    plain = [theta ** (-(2 * j) / d) for j in range(d // 2)]
    for got in (rope_inverse_frequencies(d, theta, s).double(), inverse_frequencies(d, theta, s).double()):
        band = BAND[name]
        for j, f in enumerate(got.tolist()):
            if j in band:
                assert abs(f - band[j]) <= 1e-7 * band[j]
                assert plain[j] / s["factor"] < f < plain[j]                   # strictly between the two
            elif j < min(band):
                assert abs(f - plain[j]) <= 1e-7 * plain[j]                   # fast frequencies: unchanged
            else:
                assert abs(f - plain[j] / s["factor"]) <= 1e-7 * plain[j]     # slow ones: divided
        assert all(a > b for a, b in zip(got.tolist(), got.tolist()[1:]))     # still falling with the index


def test_without_scaling_it_is_the_reference_formula():
    """include/photon/ops/kernels/rope_kernel.hpp:68-74: ``1 / 10000^(d / head_size)`` for even ``d``."""
    for d in (16, 48, 64):
        want = torch.tensor([1.0 / 10000.0 ** (2 * j / d) for j in range(d // 2)], dtype=torch.float64)
        for got in (rope_inverse_frequencies(d, 10000.0, None), inverse_frequencies(d, 10000.0, None)):
            assert float(((got.double() - want) / want).abs().max()) < 1e-7
