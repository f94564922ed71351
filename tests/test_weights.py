"""Weights by tensor name: the one error that lists everything, dtypes, the random-weights mode."""
import json
import os
import struct

import pytest
import torch

from helpers import TINY, make_model_folder
from photon_infer_b200.config import LlamaConfig, get_architecture
from photon_infer_b200.errors import ErrorCode, PhotonError
from photon_infer_b200.models.model import declared_tensors
from photon_infer_b200.weights import load_tensors, open_model_files, write_random_model, write_safetensors
from photon_infer_b200.weights.safetensors_io import SafetensorsFile


def _declared(name):
    cfg = LlamaConfig.from_dict(TINY[name]["config"])
    return declared_tensors(get_architecture(cfg.architecture).build_spec(cfg))


def _read_all(folder):
    entries, files = open_model_files(folder)
    out = {n: e.file.read(n) for n, e in entries.items()}
    for f in files:
        f.close()
    return out


def test_random_model_folder(tmp_path):
    folder = make_model_folder(str(tmp_path), "tiny_b")
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    cfg = json.load(open(os.path.join(folder, "config.json")))
    assert cfg["architectures"] == ["LlamaForCausalLM"] and cfg["hidden_size"] == 96
    tensors = _read_all(folder)
    declared = _declared("tiny_b")
    assert set(tensors) == set(declared)
    assert "lm_head.weight" in tensors
    for n, t in tensors.items():
        assert tuple(t.shape) == declared[n].shape and t.dtype == torch.bfloat16
    w = tensors["model.layers.1.mlp.down_proj.weight"].float()
    assert abs(float(w.std()) - 0.05) < 0.005
    g = tensors["model.layers.0.input_layernorm.weight"].float()
    assert abs(float(g.mean()) - 1.0) < 0.1 and 0.03 < float(g.std()) < 0.2
    # the safetensors package reads the same file
    from safetensors.torch import load_file
    other = load_file(os.path.join(folder, "model.safetensors"))
    assert all(torch.equal(other[n], tensors[n]) for n in tensors)


def test_seed_decides_values(tmp_path):
    a = _read_all(make_model_folder(str(tmp_path / "a"), "tiny_a"))
    b = _read_all(make_model_folder(str(tmp_path / "b"), "tiny_a"))
    assert all(torch.equal(a[n], b[n]) for n in a)
    t = TINY["tiny_a"]
    write_random_model(str(tmp_path / "c"), t["config"], seed=t["seed"] + 1, init_std=t["init_std"])
    c = _read_all(str(tmp_path / "c"))
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert "lm_head.weight" not in a            # tied


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    folder = make_model_folder(str(tmp_path), "tiny_a")
    tensors = _read_all(folder)
    del tensors["model.layers.1.self_attn.k_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.7.extra.weight"] = torch.zeros(3)
    tensors["model.layers.0.mlp.up_proj.weight"] = torch.zeros(5, 64, dtype=torch.bfloat16)
    tensors["model.embed_tokens.weight"] = tensors["model.embed_tokens.weight"].to(torch.int32)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with pytest.raises(PhotonError) as e:
        load_tensors(folder, _declared("tiny_a"), torch.bfloat16, "cpu")
    msg = str(e.value)
    assert e.value.code == ErrorCode.WEIGHTS_MISMATCH
    assert "missing (2)" in msg and "model.layers.1.self_attn.k_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected (1)" in msg and "model.layers.7.extra.weight" in msg
    assert "model.layers.0.mlp.up_proj.weight: expected [128, 64], file has [5, 64]" in msg
    assert "model.embed_tokens.weight" in msg and "floating point" in msg


def test_buffers_some_exports_carry_are_skipped_with_a_warning(tmp_path, capsys):
    """Older Llama exports store every layer's rotation frequencies; the architecture names the pattern and the
    loader skips them with one line on stderr.  Any other extra tensor is still an error."""
    from photon_infer_b200.config.registry import get_architecture
    folder = make_model_folder(str(tmp_path), "tiny_a")
    arch = get_architecture("LlamaForCausalLM")
    spec = arch.build_spec(arch.config_class.from_dict(TINY["tiny_a"]["config"]))
    tensors = _read_all(folder)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    tensors["model.layers.1.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    got = load_tensors(folder, _declared("tiny_a"), torch.bfloat16, "cpu", spec.ignored_tensors)
    assert "rotary_emb.inv_freq" not in " ".join(got)
    assert "2 tensors" in capsys.readouterr().err
    with pytest.raises(PhotonError) as e:
        load_tensors(folder, _declared("tiny_a"), torch.bfloat16, "cpu")
    assert "unexpected (2)" in str(e.value)


def test_untied_model_needs_its_head(tmp_path):
    folder = make_model_folder(str(tmp_path), "tiny_b")
    tensors = _read_all(folder)
    del tensors["lm_head.weight"]
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with pytest.raises(PhotonError) as e:
        load_tensors(folder, _declared("tiny_b"), torch.float32, "cpu")
    assert "lm_head.weight" in str(e.value)


def test_storage_dtypes(tmp_path):
    """bfloat16 stays bfloat16; a vector stored in 32-bit stays 32-bit; the float32 run widens everything."""
    folder = make_model_folder(str(tmp_path), "tiny_a")
    tensors = _read_all(folder)
    name = "model.layers.0.input_layernorm.weight"
    exact = torch.full((64,), 1.0 + 2.0 ** -12)              # not representable in bfloat16
    tensors[name] = exact
    tensors["model.layers.0.mlp.down_proj.weight"] = tensors["model.layers.0.mlp.down_proj.weight"].float()
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    got = load_tensors(folder, _declared("tiny_a"), torch.bfloat16, "cpu")
    assert got[name].dtype == torch.float32 and torch.equal(got[name], exact)
    assert got["model.norm.weight"].dtype == torch.bfloat16
    assert got["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16     # a matrix runs in the run dtype
    assert got["model.embed_tokens.weight"].dtype == torch.bfloat16
    got32 = load_tensors(folder, _declared("tiny_a"), torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in got32.values())
    assert torch.equal(got32["model.embed_tokens.weight"], tensors["model.embed_tokens.weight"].float())


def test_broken_files(tmp_path):
    p = tmp_path / "model.safetensors"
    with pytest.raises(PhotonError) as e:
        open_model_files(str(tmp_path))
    assert e.value.code == ErrorCode.FILE_NOT_FOUND
    p.write_bytes(b"\x01\x02")
    with pytest.raises(PhotonError) as e:
        SafetensorsFile(str(p))
    assert e.value.code == ErrorCode.INVALID_FILE
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(PhotonError):
        SafetensorsFile(str(p))
    header = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)      # truncated data
    with pytest.raises(PhotonError) as e:
        SafetensorsFile(str(p))
    assert "offsets" in str(e.value)
    header = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 4)
    with pytest.raises(PhotonError) as e:
        SafetensorsFile(str(p))
    assert "dtype" in str(e.value)


def test_sharded_folder(tmp_path):
    folder = make_model_folder(str(tmp_path), "tiny_a")
    tensors = _read_all(folder)
    names = sorted(tensors)
    half = len(names) // 2
    write_safetensors(os.path.join(folder, "model-00001-of-00002.safetensors"), {n: tensors[n] for n in names[:half]})
    write_safetensors(os.path.join(folder, "model-00002-of-00002.safetensors"), {n: tensors[n] for n in names[half:]})
    os.remove(os.path.join(folder, "model.safetensors"))
    wm = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
          for i, n in enumerate(names)}
    json.dump({"weight_map": wm}, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    got = load_tensors(folder, _declared("tiny_a"), torch.bfloat16, "cpu")
    assert all(torch.equal(got[n], tensors[n]) for n in names)
