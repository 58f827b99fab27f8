"""Typed configuration and the architecture registry."""

import json

import pytest

from atomserve_b200.config import EngineConfig, ModelConfigError, Qwen3Config, architecture_for, load_model_config
from atomserve_b200.config.registry import config_from_dict
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_reads_every_key_and_defaults():
    arch, c = config_from_dict(TINY_B)
    assert arch.name == "Qwen3ForCausalLM" and isinstance(c, Qwen3Config)
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (512, 96, 224, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (6, 3, 32)
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 1e6 and c.tie_word_embeddings is False
    raw = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "tie_word_embeddings")}
    _, d = config_from_dict(raw)
    assert d.head_dim == 64 // 4 and d.tie_word_embeddings is False  # atomserve/config.py:55,58


def test_round_trips_through_config_json(tmp_path):
    for raw in (TINY_A, TINY_B, TINY_C):
        _, c = config_from_dict(raw)
        (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
        _, again = load_model_config(tmp_path)
        assert again == c


@pytest.mark.parametrize(
    "change,message",
    [
        (dict(architectures=["LlamaForCausalLM"]), "not registered"),
        (dict(architectures=[]), "exactly one architecture"),
        (dict(attention_bias=True), "attention_bias"),
        (dict(rope_scaling={"type": "yarn"}), "rope_scaling"),
        (dict(hidden_act="gelu"), "hidden_act"),
        (dict(num_key_value_heads=3), "multiple"),
        (dict(head_dim=15), "even"),
        (dict(use_sliding_window=True, sliding_window=0), "sliding_window"),
        (dict(num_hidden_layers=0), "positive"),
    ],
)
def test_rejections(change, message):
    with pytest.raises(ModelConfigError, match=message):
        config_from_dict({**TINY_A, **change})


def test_missing_required_key_is_named():
    raw = {k: v for k, v in TINY_A.items() if k != "rope_theta"}
    with pytest.raises(ModelConfigError, match="rope_theta"):
        config_from_dict(raw)


def test_window_layers():
    _, c = config_from_dict(TINY_C)
    assert [c.window_of_layer(i) for i in range(4)] == [None, 24, 24, 24]
    _, a = config_from_dict(TINY_A)
    assert a.window_of_layer(1) is None


def test_registry_lookup_and_spec():
    arch = architecture_for("Qwen3ForCausalLM")
    _, c = config_from_dict(TINY_C)
    spec = arch.build_spec(c)
    assert len(spec.layers) == 4 and [call.layer for call in spec.schedule] == [0, 1, 2, 3]
    assert spec.layers[0].mixer.params["window"] is None and spec.layers[2].mixer.params["window"] == 24
    assert spec.layers[1].mixer.params["num_kv_heads"] == 1 and spec.head.params["tied"] is False


def test_engine_config_checks():
    EngineConfig(num_blocks=8, block_size=16, max_model_len=128, max_num_seqs=4, max_num_batched_tokens=4)
    with pytest.raises(ValueError, match="exceeds"):
        EngineConfig(num_blocks=8, block_size=16, max_model_len=129)
    with pytest.raises(ValueError, match="max_num_batched_tokens"):
        EngineConfig(max_num_seqs=64, max_num_batched_tokens=32)
