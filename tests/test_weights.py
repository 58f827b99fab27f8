"""Loading by tensor name, the one error that lists everything wrong, and random models."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

import plain_qwen3 as plain
from atomserve_b200.config.registry import config_from_dict
from atomserve_b200.parts import build_model
from atomserve_b200.weights import WeightsError, load_model, write_model_folder
from helpers import write_folder
from tiny_configs import TINY_A, TINY_B


def test_loads_by_name_stacks_and_keeps_dtypes(tmp_path):
    w = plain.random_checkpoint(TINY_B, 1)
    folder = write_folder(TINY_B, w, tmp_path)
    _, cfg, model = load_model(folder, "bfloat16", "cpu")
    attn = model.blocks[1].mixer
    p = "model.layers.1.self_attn."
    stacked = torch.cat([w[p + f"{n}_proj.weight"] for n in "qkv"]).bfloat16()
    assert attn.qkv_proj.dtype == torch.bfloat16 and torch.equal(attn.qkv_proj, stacked)
    assert attn.q_gain.dtype == torch.float32 and torch.equal(attn.q_gain, w[p + "q_norm.weight"])
    ff = model.blocks[2].feed_forward
    p = "model.layers.2.mlp."
    assert torch.equal(ff.gate_up_proj, torch.cat([w[p + "gate_proj.weight"], w[p + "up_proj.weight"]]).bfloat16())
    assert model.head.weight is not model.embedding.table  # untied
    _, _, model32 = load_model(folder, "float32", "cpu")
    assert model32.blocks[0].mixer.o_proj.dtype == torch.float32


def test_tied_head_ignores_a_shipped_copy(tmp_path):
    w = plain.random_checkpoint(TINY_A, 1)
    w["lm_head.weight"] = torch.zeros(256, 64)  # tied checkpoints may ship one; the config decides
    folder = write_folder(TINY_A, w, tmp_path)
    _, _, model = load_model(folder, "float32", "cpu")
    assert model.head.weight is model.embedding.table


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    w = plain.random_checkpoint(TINY_B, 1)
    del w["model.layers.0.mlp.up_proj.weight"]
    del w["lm_head.weight"]
    w["model.layers.7.extra.weight"] = torch.zeros(3)
    w["model.layers.1.self_attn.k_norm.weight"] = torch.zeros(16)
    w["model.norm.weight"] = torch.zeros(96, 2)
    folder = write_folder(TINY_B, w, tmp_path)
    with pytest.raises(WeightsError) as e:
        load_model(folder, "float32", "cpu")
    text = str(e.value)
    assert "missing tensors (2)" in text and "model.layers.0.mlp.up_proj.weight" in text and "lm_head.weight" in text
    assert "unexpected tensors (1)" in text and "model.layers.7.extra.weight" in text
    assert "wrong shapes (2)" in text and "k_norm.weight: file has [16], model needs [32]" in text


def test_no_safetensors_and_no_config(tmp_path):
    with pytest.raises(FileNotFoundError, match="config.json"):
        load_model(tmp_path, "float32", "cpu")
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(FileNotFoundError, match="safetensors"):
        load_model(tmp_path, "float32", "cpu")


def test_sharded_checkpoints(tmp_path):
    w = plain.random_checkpoint(TINY_A, 2)
    names = sorted(w)
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    save_file({n: w[n] for n in names[::2]}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file({n: w[n] for n in names[1::2]}, str(tmp_path / "model-00002-of-00002.safetensors"))
    _, _, model = load_model(tmp_path, "float32", "cpu")
    assert torch.equal(model.final_norm.gain, w["model.norm.weight"])


def test_random_model_folder_is_seeded_and_loadable(tmp_path):
    _, cfg = config_from_dict(TINY_B)
    a = write_model_folder(cfg, 5, tmp_path / "a", "bfloat16", eos_token_ids=[3])
    b = write_model_folder(cfg, 5, tmp_path / "b", "bfloat16")
    c = write_model_folder(cfg, 6, tmp_path / "c", "float32")
    ta, tb, tc = (load_file(str(d / "model.safetensors")) for d in (a, b, c))
    assert set(ta) == {s.name for s in build_model(config_from_dict(TINY_B)[0].build_spec(cfg)).tensor_specs()}
    assert all(torch.equal(ta[n], tb[n]) for n in ta)
    assert not torch.equal(ta["lm_head.weight"].float(), tc["lm_head.weight"])
    assert ta["lm_head.weight"].dtype == torch.bfloat16 and ta["model.norm.weight"].dtype == torch.float32
    assert tc["lm_head.weight"].dtype == torch.float32
    assert abs(float(ta["lm_head.weight"].float().std()) - 0.02) < 0.002
    assert abs(float(ta["model.norm.weight"].mean()) - 1.0) < 0.05
    assert json.loads((a / "config.json").read_text())["architectures"] == ["Qwen3ForCausalLM"]
    assert json.loads((a / "generation_config.json").read_text()) == {"eos_token_id": [3]}
    _, cfg2, model = load_model(a, "float32", "cpu")
    assert cfg2 == cfg and model.head.weight.shape == (512, 96)
    from atomserve_b200.weights.loader import read_eos_token_ids

    assert read_eos_token_ids(a) == frozenset({3}) and read_eos_token_ids(b) == frozenset()


def test_a_tensor_held_by_two_files_is_an_error_and_an_index_decides_what_belongs(tmp_path):
    """A stale shard left in the folder must not change the weights silently: a name in two files
    is reported with the rest; where the folder has an index, only the files it names count."""
    w = plain.random_checkpoint(TINY_A, 2)
    names = sorted(w)
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    save_file({n: w[n] for n in names[::2]}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file({n: w[n] for n in names[1::2]}, str(tmp_path / "model-00002-of-00002.safetensors"))
    stale = {names[0]: w[names[0]] + 1, names[1]: w[names[1]] + 1}
    save_file(stale, str(tmp_path / "stale.safetensors"))
    with pytest.raises(WeightsError) as e:
        load_model(tmp_path, "float32", "cpu")
    text = str(e.value)
    assert "more than one file (2)" in text and f"{names[0]} (in model-00001-of-00002.safetensors, stale.safetensors)" in text
    index = {"weight_map": {n: f"model-0000{1 + i % 2}-of-00002.safetensors" for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    _, _, model = load_model(tmp_path, "float32", "cpu")
    assert torch.equal(model.final_norm.gain, w["model.norm.weight"])
    index["weight_map"]["x"] = "gone.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(FileNotFoundError, match="gone.safetensors"):
        load_model(tmp_path, "float32", "cpu")
