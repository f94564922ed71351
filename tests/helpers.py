"""Shared pieces of the tests: tiny configurations, model folders in temporary
places, the plain implementation as oracle, and a driver for ``bin/trace_run``."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")

# Tiny configurations that differ in every size and option.
TINY: Dict[str, dict] = {
    # the reference's own constants: rope base 10000, neighbouring pairs, eps 1e-5, tied head
    "tiny_a": dict(
        config=dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128,
                    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, vocab_size=256,
                    max_position_embeddings=512, rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None,
                    rope_interleaved=True, tie_word_embeddings=True, bos_token_id=1, eos_token_id=2),
        seed=0, init_std=0.02, norm_std=0.1, block_size=16),
    # one key/value head for three query heads, llama3 frequency scaling, untied head
    "tiny_b": dict(
        config=dict(architectures=["LlamaForCausalLM"], hidden_size=96, intermediate_size=200,
                    num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1, vocab_size=384,
                    max_position_embeddings=512, rms_norm_eps=1e-6, rope_theta=500000.0,
                    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                      original_max_position_embeddings=64),
                    tie_word_embeddings=False, bos_token_id=0, eos_token_id=[5, 7]),
        seed=1, init_std=0.05, norm_std=0.1, block_size=8),
    # head_dim not hidden/heads, odd vocabulary, a window on every other layer
    "tiny_c": dict(
        config=dict(architectures=["LlamaForCausalLM"], hidden_size=120, intermediate_size=176,
                    num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=2, head_dim=48,
                    vocab_size=389, max_position_embeddings=1024, rms_norm_eps=3e-6, rope_theta=250000.0,
                    rope_scaling=dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=2.0,
                                      original_max_position_embeddings=32),
                    tie_word_embeddings=False, sliding_window=24,
                    layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
                    bos_token_id=3, eos_token_id=4),
        seed=2, init_std=0.08, norm_std=0.2, block_size=16),
    # heads of 64 (the size the tensor-memory attention kernel takes), three query heads per key/value
    # head, a window on the first layer, half-split rotation pairs, pages of 32
    "tiny_d": dict(
        config=dict(architectures=["LlamaForCausalLM"], hidden_size=160, intermediate_size=208,
                    num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=64,
                    vocab_size=301, max_position_embeddings=1024, rms_norm_eps=2e-5, rope_theta=100000.0,
                    rope_scaling=None, tie_word_embeddings=True, sliding_window=40,
                    layer_types=["sliding_attention", "full_attention"], bos_token_id=1, eos_token_id=2),
        seed=3, init_std=0.06, norm_std=0.15, block_size=32),
}


def make_model_folder(path: str, name: str, dtype: str = "bfloat16") -> str:
    from photon_infer_b200.weights import write_random_model
    t = TINY[name]
    write_random_model(path, t["config"], seed=t["seed"], init_std=t["init_std"], norm_std=t["norm_std"], dtype=dtype)
    return path


def random_ids(n: int, vocab: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


_plain_cache: Dict[tuple, torch.Tensor] = {}


def plain_logits(folder: str, ids: Sequence[int], dtype=torch.float32, **kw) -> torch.Tensor:
    from plain.llama_plain import PlainLlama
    key = (folder, tuple(ids), dtype, repr(sorted(kw.items())))
    if key not in _plain_cache:
        _plain_cache[key] = PlainLlama.from_folder(folder, dtype=dtype, **kw).logits(ids)
    return _plain_cache[key]


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """Largest absolute difference over the largest absolute wanted value."""
    return float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


# float32: both sides are 32-bit with different summation orders.
# bfloat16: activations are rounded to 8 bits of mantissa at every matrix product; the bound is a few
# roundings' worth (2^-8 each) relative to the largest logit.
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}


class TraceSession:
    """Drives one ``bin/trace_run`` process: a step goes in, ``done`` comes back, logits are read."""

    def __init__(self, model: str, dtype: str, out_dir: str, max_tokens: int, block_size: int, vocab: int):
        self.out_dir = out_dir
        self.vocab = vocab
        self.step_no = 0
        env = dict(os.environ)
        self.proc = subprocess.Popen(
            [sys.executable, TRACE_RUN, "--model", model, "--dtype", dtype, "--out", out_dir,
             "--max-tokens", str(max_tokens), "--block-size", str(block_size)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)

    def step(self, entries: List[dict], end: Sequence[str] = ()) -> Optional[np.ndarray]:
        rec = {"step": self.step_no, "entries": entries, "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.strip() != f"done {self.step_no}":
            rc = self.proc.poll()
            raise RuntimeError(f"trace_run answered {line!r} to step {self.step_no} (exit code {rc})")
        path = os.path.join(self.out_dir, f"{self.step_no}.f32")
        self.step_no += 1
        wanted = sum(len(e.get("want", [])) for e in entries)
        if wanted == 0:
            assert not os.path.exists(path)
            return None
        data = np.fromfile(path, dtype="<f4")
        os.remove(path)
        return data.reshape(wanted, self.vocab)

    def close(self) -> int:
        self.proc.stdin.close()
        rc = self.proc.wait(timeout=120)
        return rc


def round64(n: int) -> int:
    return (n + 63) // 64 * 64
