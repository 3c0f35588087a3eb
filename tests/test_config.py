"""Configuration reading and the architecture registry (no GPU)."""
import copy
import json

import pytest

from helpers import TINY_A, TINY_B, TINY_C
from scriptling_llm_lib_b200 import models  # noqa: F401
from scriptling_llm_lib_b200.config import (ConfigError, LlamaConfig, architecture_for, load_config,
                                             register_architecture, registered_architectures)


def test_reads_every_size_from_config_json():
    a = LlamaConfig.from_dict(TINY_A)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (2, 64, 4, 2, 16)
    assert (a.intermediate_size, a.vocab_size, a.rope_theta, a.rms_norm_eps) == (176, 256, 10000.0, 1e-5)
    assert a.tie_word_embeddings and a.max_position_embeddings == 128 and a.rope_pairing == "interleaved"
    assert a.eos_token_ids == (7,) and a.sliding_window is None and a.rope_scaling is None and a.rotary_dim == 16
    b = LlamaConfig.from_dict(TINY_B)
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (3, 96, 3, 1, 32)
    assert b.rotary_dim == 16 and b.rope_pairing == "half" and not b.tie_word_embeddings
    assert b.rope_scaling.rope_type == "llama3" and b.rope_scaling.factor == 8.0
    assert b.rope_scaling.original_max_position_embeddings == 64 and b.eos_token_ids == (11, 12)
    c = LlamaConfig.from_dict(TINY_C)
    assert c.sliding_window == 24 and c.head_dim == 48 and c.q_width == 288 and c.kv_width == 144


def test_defaults_follow_the_reference():
    raw = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta", "rms_norm_eps",
                                                        "rope_pairing", "tie_word_embeddings", "eos_token_id")}
    c = LlamaConfig.from_dict(raw)
    assert c.num_key_value_heads == c.num_attention_heads          # gguf.go:589-590
    assert c.head_dim == c.hidden_size // c.num_attention_heads    # model_f32.go:249
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-5      # gguf.go:594-595
    assert c.rope_pairing == "half" and c.tie_word_embeddings is False and c.eos_token_ids == ()


def test_round_trip_through_json():
    for raw in (TINY_A, TINY_B, TINY_C):
        c = LlamaConfig.from_dict(raw)
        again = LlamaConfig.from_dict(json.loads(json.dumps(c.to_json_dict())))
        assert again == c


@pytest.mark.parametrize("change, word", [
    ({"hidden_size": None}, "hidden_size"), ({"vocab_size": "many"}, "vocab_size"),
    ({"num_key_value_heads": 3}, "multiple"), ({"num_hidden_layers": 0}, "at least"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"), ({"rope_pairing": "odd"}, "rope_pairing"),
    ({"partial_rotary_factor": 0.3}, "rotary"), ({"eos_token_id": 999}, "vocabulary"),
    ({"rms_norm_eps": -1.0}, "positive"), ({"architectures": []}, "architectures"),
    ({"hidden_size": 65, "head_dim": None}, "head_dim"),
])
def test_bad_configs_name_the_key(change, word):
    raw = copy.deepcopy(TINY_A)
    raw.update(change)
    raw = {k: v for k, v in raw.items() if not (v is None and k in ("hidden_size",))}
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(raw)
    assert word in str(e.value)


def test_unknown_keys_are_reported_not_fatal():
    raw = dict(TINY_A, some_future_key=3)
    assert LlamaConfig.from_dict(raw).unknown_keys == ("some_future_key",)


def test_registry(tmp_path):
    assert "LlamaForCausalLM" in registered_architectures()
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    arch, cfg = load_config(tmp_path)
    assert arch.name == "LlamaForCausalLM" and isinstance(cfg, LlamaConfig)
    layout = arch.layout(cfg)
    assert len(layout.layers) == 3 and layout.stop_ids == (11, 12)
    assert layout.head.kind == "linear_head" and layout.head.params["weight_name"] == "lm_head.weight" and not layout.head.params["tied"]
    assert layout.embedding.kind == "token_embedding" and layout.layers[0].arrangement == "pre_norm"
    assert layout.layers[0].parts["mixer"].kind == "attention" and layout.layers[0].parts["feed_forward"].kind == "swiglu"
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_B, architectures=["NopeForCausalLM"])))
    with pytest.raises(ConfigError) as e:
        load_config(tmp_path)
    assert "NopeForCausalLM" in str(e.value) and "LlamaForCausalLM" in str(e.value)
    with pytest.raises(ValueError):
        register_architecture("LlamaForCausalLM", LlamaConfig, lambda c: None)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(tmp_path)
    with pytest.raises(ConfigError):
        load_config(tmp_path / "nowhere")
    assert architecture_for("LlamaForCausalLM").config_class is LlamaConfig
