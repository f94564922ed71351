"""Configuration from config.json keys, and the registry from architecture name to model."""
import json

import pytest

from helpers import TINY
from photon_infer_b200.config import LlamaConfig, get_architecture, load_config, register_architecture, registered_architectures
from photon_infer_b200.errors import ErrorCode, PhotonError

BASE = TINY["tiny_b"]["config"]


def test_reads_every_key():
    c = LlamaConfig.from_dict(BASE)
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (96, 200, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (3, 1, 32)
    assert c.vocab_size == 384 and c.max_position_embeddings == 512
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 500000.0
    assert c.rope_scaling.rope_type == "llama3" and c.rope_scaling.factor == 8.0
    assert c.rope_scaling.original_max_position_embeddings == 64
    assert not c.tie_word_embeddings and c.eos_token_ids == (5, 7) and c.bos_token_id == 0
    assert c.layer_types == ("full_attention",) * 3 and c.sliding_window is None


def test_defaults_are_the_references_constants():
    d = {k: v for k, v in BASE.items() if k not in ("rms_norm_eps", "rope_theta", "rope_scaling", "num_key_value_heads")}
    c = LlamaConfig.from_dict(d)
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0 and c.rope_scaling is None
    assert c.num_key_value_heads == c.num_attention_heads


def test_head_dim_key_overrides_the_quotient():
    c = LlamaConfig.from_dict(TINY["tiny_c"]["config"])
    assert c.head_dim == 48 and c.hidden_size // c.num_attention_heads == 20
    assert c.layer_types[0] == "sliding_attention" and c.sliding_window == 24


def test_round_trip():
    for t in TINY.values():
        c = LlamaConfig.from_dict(t["config"])
        assert LlamaConfig.from_dict(json.loads(json.dumps(c.to_dict()))) == c


@pytest.mark.parametrize("change,needle", [
    ({"hidden_size": None}, "hidden_size"),
    ({"vocab_size": "big"}, "vocab_size"),
    ({"num_key_value_heads": 2}, "num_key_value_heads"),
    ({"head_dim": 15}, "head_dim"),
    ({"hidden_size": 100}, "head_dim"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "rope_type"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "low_freq_factor"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"layer_types": ["sliding_attention"] * 3}, "sliding_window"),
    ({"eos_token_id": "x"}, "eos_token_id"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"architectures": []}, "architectures"),
    ({"rms_norm_eps": -1.0}, "rms_norm_eps"),
])
def test_errors_name_the_key(change, needle):
    d = dict(BASE)
    d.update(change)
    if change.get("hidden_size") == 100:
        d.pop("head_dim", None)
    with pytest.raises(PhotonError) as e:
        LlamaConfig.from_dict(d)
    assert needle in str(e.value)
    assert e.value.code == ErrorCode.INVALID_CONFIG


@pytest.mark.parametrize("change", [{"attention_bias": True}, {"mlp_bias": True}, {"hidden_act": "gelu"}])
def test_unsupported_options(change):
    with pytest.raises(PhotonError) as e:
        LlamaConfig.from_dict(dict(BASE, **change))
    assert e.value.code == ErrorCode.UNSUPPORTED_MODEL


def test_registry(tmp_path):
    assert "LlamaForCausalLM" in registered_architectures()
    with pytest.raises(PhotonError) as e:
        get_architecture("NoSuchModel")
    assert e.value.code == ErrorCode.UNSUPPORTED_MODEL and "LlamaForCausalLM" in str(e.value)
    (tmp_path / "config.json").write_text(json.dumps(BASE))
    arch, cfg = load_config(str(tmp_path))
    assert arch.name == "LlamaForCausalLM" and isinstance(cfg, LlamaConfig)
    spec = arch.build_spec(cfg)
    assert len(spec.layers) == 3 and [e.layer for e in spec.run] == [0, 1, 2]
    assert spec.head_name == "lm_head.weight"
    (tmp_path / "config.json").write_text(json.dumps(dict(BASE, architectures=["Other"])))
    with pytest.raises(PhotonError):
        load_config(str(tmp_path))
    with pytest.raises(PhotonError) as e:
        load_config(str(tmp_path / "nowhere"))
    assert e.value.code == ErrorCode.FILE_NOT_FOUND
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(PhotonError) as e:
        load_config(str(tmp_path))
    assert e.value.code == ErrorCode.INVALID_FILE


def test_register_twice_is_refused():
    with pytest.raises(PhotonError):
        register_architecture("LlamaForCausalLM", LlamaConfig, lambda c: None)


def test_spec_takes_no_size_from_code():
    """Every size in the spec changes when its key changes."""
    a = get_architecture("LlamaForCausalLM")
    s1 = a.build_spec(LlamaConfig.from_dict(TINY["tiny_a"]["config"]))
    s2 = a.build_spec(LlamaConfig.from_dict(TINY["tiny_c"]["config"]))
    m1, m2 = s1.layers[0].mixer.params, s2.layers[0].mixer.params
    for key in ("hidden_size", "n_q_heads", "head_dim"):
        assert m1[key] != m2[key]
    assert m1["window"] is None and m2["window"] == 24 and s2.layers[1].mixer.params["window"] is None
    assert s1.layers[0].norm1.params["eps"] != s2.layers[0].norm1.params["eps"]
    assert s1.position_encodings["rope"].params["theta"] != s2.position_encodings["rope"].params["theta"]
    assert s1.position_encodings["rope"].params["interleaved"] and not s2.position_encodings["rope"].params["interleaved"]
    assert s1.head_name is None and s2.head_name == "lm_head.weight"
