"""Typed configuration of the Llama decoder, read from the keys of its ``config.json``.

The reference fills a ``TransformerConfig`` from a 7-integer binary header
(include/photon/arch/config.hpp:16-54, src/arch/config.cpp:13-49) and fixes the rest
in code: ``norm_eps = 1e-5`` (src/io/checkpoint.cpp:117), rope base 10000
(include/photon/ops/kernels/rope_kernel.hpp:70-72), ``head_size = dim / n_heads``
(src/arch/config.cpp:29).  Here every one of those is a key; the reference's fixed
values remain only as the defaults of keys that a file leaves out.

Keys beyond the usual Llama set, all optional:

``rope_interleaved``  true selects the reference's pairing of neighbours
                      ``(x[2j], x[2j+1])``; false (default) pairs ``(x[j], x[j+d/2])``,
                      the layout of Hugging Face weight files.
``sliding_window``    window length of the layers whose ``layer_types`` entry is
                      ``"sliding_attention"``.
``layer_types``       one mixer name per layer (default: ``"full_attention"`` for all);
                      any name registered in ``parts.registry.MIXERS`` is accepted.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Dict, Optional, Tuple

from ..errors import ErrorCode, PhotonError

_MISSING = object()


def _bad(msg: str) -> PhotonError:
    return PhotonError(ErrorCode.INVALID_CONFIG, msg)


def _get(d: Dict[str, Any], key: str, kind, default=_MISSING):
    """One key, type-checked; the key name is part of every error."""
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise _bad(f"config.json: required key '{key}' is missing")
        return default
    v = d[key]
    if kind is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if kind is int and isinstance(v, bool) or not isinstance(v, kind):
        raise _bad(f"config.json: key '{key}' must be {kind.__name__}, got {v!r}")
    return v


@dataclasses.dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of config.json; only ``rope_type == "llama3"`` changes frequencies."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @classmethod
    def from_dict(cls, d: Optional[Dict[str, Any]]) -> Optional["RopeScaling"]:
        if d is None:
            return None
        if not isinstance(d, dict):
            raise _bad("config.json: key 'rope_scaling' must be an object or null")
        kind = d.get("rope_type", d.get("type"))
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise _bad(f"config.json: rope_scaling.rope_type {kind!r} is not supported (llama3 or default)")
        s = cls(kind,
                _get(d, "factor", float),
                _get(d, "low_freq_factor", float),
                _get(d, "high_freq_factor", float),
                _get(d, "original_max_position_embeddings", int))
        if s.factor <= 0 or s.high_freq_factor <= s.low_freq_factor or s.low_freq_factor <= 0:
            raise _bad("config.json: rope_scaling needs factor > 0 and high_freq_factor > low_freq_factor > 0")
        if s.original_max_position_embeddings <= 0:
            raise _bad("config.json: rope_scaling.original_max_position_embeddings must be positive")
        return s

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)


@dataclasses.dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    rope_interleaved: bool
    tie_word_embeddings: bool
    hidden_act: str
    bos_token_id: Optional[int]
    eos_token_ids: Tuple[int, ...]
    torch_dtype: str
    sliding_window: Optional[int]
    layer_types: Tuple[str, ...]

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        archs = d.get("architectures")
        if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
            raise _bad("config.json: key 'architectures' must be a non-empty list of names")
        hidden = _get(d, "hidden_size", int)
        heads = _get(d, "num_attention_heads", int)
        kv_heads = _get(d, "num_key_value_heads", int, heads)
        layers = _get(d, "num_hidden_layers", int)
        for key, v in (("hidden_size", hidden), ("num_attention_heads", heads),
                       ("num_key_value_heads", kv_heads), ("num_hidden_layers", layers)):
            if v <= 0:
                raise _bad(f"config.json: key '{key}' must be positive, got {v}")
        if "head_dim" in d and d["head_dim"] is not None:
            head_dim = _get(d, "head_dim", int)
        else:
            if hidden % heads:
                raise _bad("config.json: 'hidden_size' is not a multiple of 'num_attention_heads' "
                           "and no 'head_dim' is given")
            head_dim = hidden // heads      # the reference's rule, src/arch/config.cpp:29
        if head_dim <= 0 or head_dim % 2:
            raise _bad(f"config.json: 'head_dim' must be positive and even, got {head_dim}")
        if heads % kv_heads:
            raise _bad(f"config.json: 'num_attention_heads' ({heads}) is not a multiple of "
                       f"'num_key_value_heads' ({kv_heads})")
        if _get(d, "attention_bias", bool, False):
            raise PhotonError(ErrorCode.UNSUPPORTED_MODEL, "config.json: 'attention_bias' true is not supported")
        if _get(d, "mlp_bias", bool, False):
            raise PhotonError(ErrorCode.UNSUPPORTED_MODEL, "config.json: 'mlp_bias' true is not supported")
        act = _get(d, "hidden_act", str, "silu")
        if act != "silu":
            raise PhotonError(ErrorCode.UNSUPPORTED_MODEL, f"config.json: 'hidden_act' {act!r} is not supported (silu)")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise _bad("config.json: key 'eos_token_id' must be an integer or a list of integers")
        window = _get(d, "sliding_window", int, None)
        if window is not None and window <= 0:
            raise _bad("config.json: key 'sliding_window' must be positive")
        types = d.get("layer_types")
        if types is None:
            types = ["full_attention"] * layers
        if not isinstance(types, list) or len(types) != layers or not all(isinstance(t, str) for t in types):
            raise _bad(f"config.json: key 'layer_types' must list one name for each of the {layers} layers")
        if "sliding_attention" in types and window is None:
            raise _bad("config.json: 'layer_types' names sliding_attention but 'sliding_window' is missing")
        cfg = cls(
            architecture=archs[0],
            hidden_size=hidden,
            intermediate_size=_get(d, "intermediate_size", int),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=_get(d, "vocab_size", int),
            max_position_embeddings=_get(d, "max_position_embeddings", int),
            rms_norm_eps=_get(d, "rms_norm_eps", float, 1e-5),
            rope_theta=_get(d, "rope_theta", float, 10000.0),
            rope_scaling=RopeScaling.from_dict(d.get("rope_scaling")),
            rope_interleaved=_get(d, "rope_interleaved", bool, False),
            tie_word_embeddings=_get(d, "tie_word_embeddings", bool, False),
            hidden_act=act,
            bos_token_id=_get(d, "bos_token_id", int, None),
            eos_token_ids=eos_ids,
            torch_dtype=_get(d, "torch_dtype", str, "bfloat16"),
            sliding_window=window,
            layer_types=tuple(types),
        )
        for key in ("intermediate_size", "vocab_size", "max_position_embeddings"):
            if getattr(cfg, key) <= 0:
                raise _bad(f"config.json: key '{key}' must be positive, got {getattr(cfg, key)}")
        if cfg.rms_norm_eps <= 0 or cfg.rope_theta <= 0:
            raise _bad("config.json: 'rms_norm_eps' and 'rope_theta' must be positive")
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "LlamaConfig":
        return cls.from_dict(read_config_json(path))

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "rope_interleaved": self.rope_interleaved,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": False,
            "mlp_bias": False,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": list(self.eos_token_ids) if len(self.eos_token_ids) != 1 else self.eos_token_ids[0],
            "torch_dtype": self.torch_dtype,
        }
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
        if any(t != "full_attention" for t in self.layer_types):
            d["layer_types"] = list(self.layer_types)
        return d


def read_config_json(path: str) -> Dict[str, Any]:
    """``path`` is a ``config.json`` or a folder that holds one."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if not os.path.isfile(path):
        raise PhotonError(ErrorCode.FILE_NOT_FOUND, f"no config.json at {path}")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise PhotonError(ErrorCode.INVALID_FILE, f"{path} is not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise PhotonError(ErrorCode.INVALID_FILE, f"{path} must hold a JSON object")
    return d
