"""Safetensors in and out, the whole-checkpoint check and the random-weights mode (no GPU)."""
import json

import pytest
import torch

import tiny
from plain import llama_plain as P
from spissa_b200.config import config_from_dict
from spissa_b200.engine.model import Model
from spissa_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_tensors, random_tensors,
                                 write_random_model, write_safetensors)


def specs_of(cfg_dict):
    return Model(config_from_dict(cfg_dict).to_spec()).weight_specs()


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5).bfloat16(), "b": torch.randn(7), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
         "d": torch.randn(2, 2).half(), "e": torch.tensor(3.5)}
    write_safetensors(tmp_path / "x.safetensors", t, metadata={"k": 1})
    with SafetensorsFile(tmp_path / "x.safetensors") as f:
        assert sorted(f.names()) == sorted(t) and f.metadata == {"k": "1"}
        for k, v in t.items():
            got = f.tensor(k)
            assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v)
    # the plain implementation's own reader agrees
    mine = P.read_safetensors(tmp_path / "x.safetensors")
    assert all(torch.equal(mine[k], t[k]) for k in t)


def test_bad_files_are_refused(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)
    p.write_bytes((10 ** 12).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="not plausible"):
        SafetensorsFile(p)
    with pytest.raises(FileNotFoundError):
        SafetensorsFile(tmp_path / "none.safetensors")


def test_random_model_folder_is_reproducible_and_loads(tmp_path):
    cfg = config_from_dict(tiny.TINY_B)
    a = write_random_model(cfg, tmp_path / "a", seed=3, norm_std=0.1)
    b = write_random_model(cfg, tmp_path / "b", seed=3, norm_std=0.1)
    c = write_random_model(cfg, tmp_path / "c", seed=4, norm_std=0.1)
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
    assert json.loads((a / "config.json").read_text())["architectures"] == ["LlamaForCausalLM"]
    tensors = load_tensors(a, specs_of(tiny.TINY_B), "cpu", full_precision=False)
    assert tensors["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16
    w = tensors["model.layers.2.mlp.up_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.002
    n = tensors["model.norm.weight"].float()
    assert 0.03 < float((n - 1).std()) < 0.3
    full = load_tensors(a, specs_of(tiny.TINY_B), "cpu", full_precision=True)
    assert all(v.dtype == torch.float32 for v in full.values())
    assert torch.equal(full["model.norm.weight"], n)          # widening is exact


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    specs = specs_of(tiny.TINY_A)
    tensors = random_tensors(specs, seed=1)
    del tensors["model.layers.0.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64).bfloat16()
    tensors["lm_head.weight"] = torch.zeros(256, 64).bfloat16()          # config says tied
    tensors["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(64, 64).bfloat16()
    tensors["model.layers.1.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    write_safetensors(tmp_path / "model.safetensors", tensors)
    (tmp_path / "config.json").write_text(json.dumps(tiny.TINY_A))
    with pytest.raises(WeightError) as ei:
        load_tensors(tmp_path, specs, "cpu", False)
    e = ei.value
    assert e.missing == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["lm_head.weight", "model.layers.0.self_attn.q_proj.bias"]
    assert len(e.mismatched) == 2
    text = str(e)
    for needle in ("model.norm.weight", "q_proj.bias", "[64, 64]", "[32, 64]", "stored as I32"):
        assert needle in text


def test_storage_types(tmp_path):
    specs = specs_of(tiny.TINY_A)
    tensors = random_tensors(specs, seed=1)
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()                 # stored in 32-bit: stays
    tensors["model.layers.0.mlp.up_proj.weight"] = tensors["model.layers.0.mlp.up_proj.weight"].half()
    write_safetensors(tmp_path / "model.safetensors", tensors)
    got = load_tensors(tmp_path, specs, "cpu", False)
    assert got["model.norm.weight"].dtype == torch.float32
    assert got["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert got["model.embed_tokens.weight"].dtype == torch.bfloat16


def test_sharded_index(tmp_path):
    specs = specs_of(tiny.TINY_A)
    tensors = random_tensors(specs, seed=2)
    names = sorted(tensors)
    half = len(names) // 2
    write_safetensors(tmp_path / "s1.safetensors", {n: tensors[n] for n in names[:half]})
    write_safetensors(tmp_path / "s2.safetensors", {n: tensors[n] for n in names[half:]})
    index = {"weight_map": {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    got = load_tensors(tmp_path, specs, "cpu", False)
    assert all(torch.equal(got[n], tensors[n]) for n in names)


def test_missing_model_file(tmp_path):
    with pytest.raises(FileNotFoundError, match="model.safetensors"):
        load_tensors(tmp_path, specs_of(tiny.TINY_A), "cpu", False)
