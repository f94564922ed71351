"""Plain, slow implementation of the Llama decoder: the oracle of the test suite.

Whole sequences, no cache, no batching, one function per part, torch on the CPU.
It shares no code with ``photon_infer_b200``: it reads ``config.json`` as a plain
dict and the weights with the ``safetensors`` package.

Every function cites the lines of lumia431/photon_infer that give its formula
(paths are relative to that project's root).  Where that project has no
counterpart (config.json keys, llama3 frequency scaling, the half-split pair
convention of Hugging Face weight files, a sliding window) the docstring says so
and states the formula itself.

``tests/golden/`` holds logits that the reference's own CPU kernels produced on a
tiny random model; ``tests/test_plain_reference.py`` compares this file with them.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------- parts


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """``x[t, :] = E[ids[t], :]`` with a bounds check.

    include/photon/ops/kernels/embedding_kernel.hpp:85-121 (row copy, ids outside
    ``[0, vocab)`` are an error on the CPU path).
    """
    if ids.numel() and (int(ids.min()) < 0 or int(ids.max()) >= table.shape[0]):
        raise IndexError("token id outside the vocabulary")
    return table[ids.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``y_i = w_i * (x_i / sqrt(mean(x^2) + eps))``.

    include/photon/ops/kernels/rmsnorm_kernel.hpp:71-86 (sum of squares, mean,
    ``1/sqrt(mean + eps)``, then ``weight * (x * rsqrt)``).
    """
    mean_sq = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    inv = 1.0 / torch.sqrt(mean_sq + eps)
    return weight * (x * inv)


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``y = x @ W^T`` with ``W`` stored ``[out, in]`` and no bias.

    include/photon/ops/kernels/matmul_kernel.hpp:104-129 (``output[b, m] = sum_n
    input[b, n] * weight[m, n]``).
    """
    return x @ weight.t()


def rope_inverse_frequencies(head_dim: int, theta: float,
                             scaling: Optional[dict]) -> torch.Tensor:
    """``inv_freq[j] = theta^(-2j / head_dim)`` for ``j`` in ``[0, head_dim/2)``.

    include/photon/ops/kernels/rope_kernel.hpp:68-74 computes ``1 / 10000^(d /
    head_size)`` for the even ``d = 2j`` that are used; the base 10000 is fixed
    there, here it is ``rope_theta`` of config.json.

    The reference has no frequency scaling.  ``rope_scaling`` with ``rope_type``
    ``"llama3"`` follows the published Llama 3.1 rule: with wavelength ``lam =
    2*pi / inv_freq`` and ``orig = original_max_position_embeddings``,
    ``lam > orig / low_freq_factor`` gives ``inv_freq / factor``;
    ``lam < orig / high_freq_factor`` leaves it unchanged; in between
    ``s = (orig / lam - low) / (high - low)`` and
    ``inv_freq' = (1 - s) * inv_freq / factor + s * inv_freq``.
    Computed in float64, returned in float32.
    """
    j = torch.arange(0, head_dim, 2, dtype=torch.float64)
    inv_freq = 1.0 / (float(theta) ** (j / head_dim))
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind == "llama3":
            factor = float(scaling["factor"])
            low = float(scaling["low_freq_factor"])
            high = float(scaling["high_freq_factor"])
            orig = float(scaling["original_max_position_embeddings"])
            lam = 2.0 * math.pi / inv_freq
            smooth = (orig / lam - low) / (high - low)
            mixed = (1.0 - smooth) * inv_freq / factor + smooth * inv_freq
            inv_freq = torch.where(lam > orig / low, inv_freq / factor,
                                   torch.where(lam < orig / high, inv_freq, mixed))
        elif kind not in (None, "default"):
            raise ValueError(f"rope_type {kind!r} is not known to the plain implementation")
    return inv_freq.to(torch.float32)


def rope_apply(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
               interleaved: bool) -> torch.Tensor:
    """Rotate the pairs of every head of ``x[T, heads, head_dim]``.

    include/photon/ops/kernels/rope_kernel.hpp:143-165: the pair ``(x0, x1)``
    becomes ``(x0*cos - x1*sin, x0*sin + x1*cos)`` with the angle ``pos *
    inv_freq[j]`` computed in 32-bit (``:76-82``).  The reference pairs the
    neighbours ``(x[2j], x[2j+1])`` (``interleaved=True``).  Weight files in the
    Hugging Face layout pair ``(x[j], x[j + head_dim/2])`` instead
    (``interleaved=False``); the rotation itself is the same.
    """
    angle = positions.to(torch.float32)[:, None] * inv_freq[None, :]     # 32-bit product
    cos = torch.cos(angle).to(x.dtype)[:, None, :]
    sin = torch.sin(angle).to(x.dtype)[:, None, :]
    out = torch.empty_like(x)
    if interleaved:
        x0, x1 = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = x0 * cos - x1 * sin
        out[..., 1::2] = x0 * sin + x1 * cos
    else:
        half = x.shape[-1] // 2
        x0, x1 = x[..., :half], x[..., half:]
        out[..., :half] = x0 * cos - x1 * sin
        out[..., half:] = x0 * sin + x1 * cos
    return out


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     window: Optional[int] = None) -> torch.Tensor:
    """Dense causal attention with grouped heads over one whole sequence.

    include/photon/ops/kernels/mha_kernel.hpp:188-229: head ``h`` uses key/value
    head ``h / (n_q / n_kv)``; ``score_t = (q . k_t) / sqrt(head_dim)`` for the
    keys ``t <= pos`` only; softmax as ``exp(s - max) / sum`` (``:36-55``, no
    epsilon in the denominator); output ``sum_t p_t * v_t``.

    ``window`` (not in the reference): the query at position ``p`` sees the keys
    ``p - window < t <= p``.

    ``q`` is ``[T, n_q, d]``, ``k`` and ``v`` are ``[T, n_kv, d]``; returns ``[T, n_q, d]``.
    """
    T, n_q, d = q.shape
    n_kv = k.shape[1]
    group = n_q // n_kv
    scale = 1.0 / math.sqrt(d)
    out = torch.zeros_like(q)
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= pos[None, :] > (pos[:, None] - window)
    for h in range(n_q):
        g = h // group
        scores = (q[:, h, :] @ k[:, g, :].t()) * scale
        scores = scores.masked_fill(~visible, float("-inf"))
        m = scores.max(dim=-1, keepdim=True).values
        e = torch.exp(scores - m)
        p = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, g, :]
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``(g / (1 + exp(-g))) * u``.

    include/photon/ops/kernels/swiglu_kernel.hpp:67-76.
    """
    return (gate / (1.0 + torch.exp(-gate))) * up


def feed_forward(h: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
                 w_down: torch.Tensor) -> torch.Tensor:
    """``down(swiglu(gate(h), up(h)))``.

    src/arch/transformer_block.cpp:282-291 (``w1`` is the gate, ``w3`` the up and
    ``w2`` the down projection).
    """
    return linear(swiglu(linear(h, w_gate), linear(h, w_up)), w_down)


# --------------------------------------------------------------------------- model


class PlainLlama:
    """Llama decoder over a whole sequence: ``logits(ids) -> [T, vocab]``.

    Block order as src/arch/transformer_block.cpp:199-296: norm, q/k/v, rotation of
    q and k, attention over all earlier keys, output projection, residual add,
    norm, feed-forward, residual add; then src/arch/llama_model.cpp:248-255: final
    norm and the output head (the embedding table when tied,
    src/io/checkpoint.cpp:305-313).

    ``layer_order`` (default ``0..L-1``) lists the layers in the order they run; a
    layer may appear twice.  ``kv_source`` maps an index of that list to an earlier
    index whose rotated keys and values the entry reads instead of making its own.
    """

    def __init__(self, config: dict, weights: Dict[str, torch.Tensor],
                 dtype: torch.dtype = torch.float32,
                 layer_order: Optional[Sequence[int]] = None,
                 kv_source: Optional[Dict[int, int]] = None):
        self.cfg = config
        self.dtype = dtype
        self.w = {k: v.to(dtype) for k, v in weights.items()}
        c = config
        self.n_layers = c["num_hidden_layers"]
        self.n_q = c["num_attention_heads"]
        self.n_kv = c.get("num_key_value_heads") or self.n_q
        self.head_dim = c.get("head_dim") or c["hidden_size"] // self.n_q
        self.eps = c.get("rms_norm_eps", 1e-5)
        self.interleaved = bool(c.get("rope_interleaved", False))
        self.inv_freq = rope_inverse_frequencies(
            self.head_dim, c.get("rope_theta", 10000.0), c.get("rope_scaling"))
        types = c.get("layer_types") or ["full_attention"] * self.n_layers
        self.windows = [c.get("sliding_window") if t == "sliding_attention" else None
                        for t in types]
        self.layer_order = list(layer_order) if layer_order is not None else list(range(self.n_layers))
        self.kv_source = dict(kv_source or {})

    @classmethod
    def from_folder(cls, folder: str, dtype: torch.dtype = torch.float32, **kw) -> "PlainLlama":
        from safetensors.torch import load_file
        with open(os.path.join(folder, "config.json")) as f:
            config = json.load(f)
        weights = load_file(os.path.join(folder, "model.safetensors"))
        return cls(config, weights, dtype=dtype, **kw)

    def _attention_part(self, layer: int, h: torch.Tensor, positions: torch.Tensor,
                        shared_kv):
        p = f"model.layers.{layer}.self_attn."
        T = h.shape[0]
        q = linear(h, self.w[p + "q_proj.weight"]).view(T, self.n_q, self.head_dim)
        q = rope_apply(q, positions, self.inv_freq, self.interleaved)
        if shared_kv is None:
            k = linear(h, self.w[p + "k_proj.weight"]).view(T, self.n_kv, self.head_dim)
            v = linear(h, self.w[p + "v_proj.weight"]).view(T, self.n_kv, self.head_dim)
            k = rope_apply(k, positions, self.inv_freq, self.interleaved)
        else:
            k, v = shared_kv
        a = causal_attention(q, k, v, window=self.windows[layer])
        return linear(a.reshape(T, -1), self.w[p + "o_proj.weight"]), (k, v)

    def hidden_states(self, ids: Sequence[int]) -> torch.Tensor:
        ids_t = torch.as_tensor(list(ids), dtype=torch.long)
        positions = torch.arange(len(ids_t))
        x = embedding(ids_t, self.w["model.embed_tokens.weight"])
        kv_of_entry = {}
        for entry, layer in enumerate(self.layer_order):
            pre = f"model.layers.{layer}."
            h = rms_norm(x, self.w[pre + "input_layernorm.weight"], self.eps)
            shared = kv_of_entry[self.kv_source[entry]] if entry in self.kv_source else None
            o, kv = self._attention_part(layer, h, positions, shared)
            kv_of_entry[entry] = kv
            x = x + o
            h2 = rms_norm(x, self.w[pre + "post_attention_layernorm.weight"], self.eps)
            x = x + feed_forward(h2, self.w[pre + "mlp.gate_proj.weight"],
                                 self.w[pre + "mlp.up_proj.weight"],
                                 self.w[pre + "mlp.down_proj.weight"])
        return rms_norm(x, self.w["model.norm.weight"], self.eps)

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        y = self.hidden_states(ids)
        if self.cfg.get("tie_word_embeddings", False):
            head = self.w["model.embed_tokens.weight"]
        else:
            head = self.w["lm_head.weight"]
        return linear(y, head).to(torch.float32)

    def greedy(self, prompt: Sequence[int], max_new_tokens: int) -> List[int]:
        """Recompute the whole sequence for every new token and take the first maximum."""
        ids = list(prompt)
        out: List[int] = []
        for _ in range(max_new_tokens):
            nxt = argmax_first(self.logits(ids)[-1])
            out.append(nxt)
            ids.append(nxt)
        return out


# --------------------------------------------------------------------------- sampling


def argmax_first(logits: torch.Tensor) -> int:
    """Index of the first maximum.

    src/arch/llama_model.cpp:304-328 (linear scan, strict ``>`` keeps the earliest).
    """
    best, best_i = float("-inf"), 0
    vals = logits.tolist()
    for i, v in enumerate(vals):
        if v > best:
            best, best_i = v, i
    return best_i


def temperature_probabilities(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """``p_i = exp((l_i - max) / T) / sum`` in 32-bit.

    demo/llama_infer.cpp:78-90.
    """
    l = logits.to(torch.float32)
    e = torch.exp((l - l.max()) / temperature)
    return e / e.sum()


def inverse_cdf_sample(probs: torch.Tensor, u: float) -> int:
    """First index whose running sum reaches ``u``.

    demo/llama_infer.cpp:92-101 (``rand_val <= cumulative``); the last index when
    rounding leaves the total below ``u``.
    """
    cum = 0.0
    vals = probs.tolist()
    for i, p in enumerate(vals):
        cum += p
        if u <= cum:
            return i
    return len(vals) - 1
