"""Typed configuration and the architecture registry (no GPU)."""
import json

import pytest

from inference_bench_b200 import models  # noqa: F401
from inference_bench_b200.config import ConfigError
from inference_bench_b200.config.qwen3 import Qwen3Config
from inference_bench_b200.config.spec import read_config_json
from inference_bench_b200.engine.model import plan_from_config
from inference_bench_b200.registry import known_architectures, resolve
from tiny_configs import CONFIGS

# config.json of Qwen3-0.6B as published (it carries tie_word_embeddings=true)
QWEN3_0_6B = {
    "architectures": ["Qwen3ForCausalLM"], "attention_bias": False, "attention_dropout": 0.0, "bos_token_id": 151643, "eos_token_id": 151645,
    "head_dim": 128, "hidden_act": "silu", "hidden_size": 1024, "initializer_range": 0.02, "intermediate_size": 3072,
    "max_position_embeddings": 40960, "max_window_layers": 28, "model_type": "qwen3", "num_attention_heads": 16, "num_hidden_layers": 28,
    "num_key_value_heads": 8, "rms_norm_eps": 1e-06, "rope_scaling": None, "rope_theta": 1000000, "sliding_window": None,
    "tie_word_embeddings": True, "torch_dtype": "bfloat16", "transformers_version": "4.51.0", "use_cache": True, "use_sliding_window": False,
    "vocab_size": 151936}


def test_real_config_and_derived_sizes():
    c = Qwen3Config.from_dict(QWEN3_0_6B)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (1024, 28, 16, 8, 128)
    assert c.q_dim == 2048 and c.kv_dim == 1024 and c.qkv_rows == 4096      # head_dim is decoupled from hidden/heads
    assert c.tie_word_embeddings and c.rope_theta == 1e6 and c.sliding_window is None
    assert all(c.window_of(i) is None for i in range(28))
    cfg, plan = plan_from_config(QWEN3_0_6B)
    assert len(plan.layers) == 28 and [e.layer for e in plan.schedule] == list(range(28))
    assert plan.head.params["tied_to"] == "model.embed_tokens.weight" and plan.ignored_tensors == ("lm_head.weight",)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_tiny_configs_round_trip(name):
    raw = CONFIGS[name]["config"]
    c = Qwen3Config.from_dict(raw)
    again = Qwen3Config.from_dict(json.loads(json.dumps(c.to_dict())))
    assert again == c
    for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim"):
        assert getattr(c, key) == raw[key]
    _, plan = plan_from_config(raw)
    for i, layer in enumerate(plan.layers):
        assert layer.mixer.params["window"] == c.window_of(i)
        assert layer.mixer.params["head_dim"] == raw["head_dim"] and layer.feed_forward.params["intermediate"] == raw["intermediate_size"]
        assert layer.mixer_norm.params["eps"] == raw["rms_norm_eps"] and layer.mixer.params["position"].params["theta"] == raw["rope_theta"]


def test_defaults_and_alternate_keys():
    raw = dict(CONFIGS["A"]["config"])
    del raw["head_dim"], raw["num_key_value_heads"], raw["rope_theta"]
    raw["rope_parameters"] = {"rope_type": "default", "rope_theta": 12345.0}
    c = Qwen3Config.from_dict(raw)
    assert c.head_dim == 16 and c.num_key_value_heads == 4 and c.rope_theta == 12345.0
    nested = {"architectures": ["Qwen3ForCausalLM"], "text_config": CONFIGS["B"]["config"]}
    assert Qwen3Config.from_dict(nested).hidden_size == 96


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "rms_norm_eps", "rope_theta"])
def test_missing_key_is_named(key):
    raw = dict(CONFIGS["A"]["config"])
    del raw[key]
    with pytest.raises(ConfigError, match=f"no {key}"):
        Qwen3Config.from_dict(raw)


@pytest.mark.parametrize("change,match", [
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"layer_types": ["full_attention"]}, "names 1 layers"),
    ({"layer_types": ["sliding_attention", "full_attention"]}, "sliding_window"),
    ({"layer_types": ["linear_attention", "full_attention"]}, "not supported"),
    ({"torch_dtype": "float8_e4m3fn"}, "torch_dtype"),
    ({"num_hidden_layers": 0}, "positive"),
])
def test_refusals(change, match):
    raw = dict(CONFIGS["A"]["config"])
    raw.update(change)
    with pytest.raises(ConfigError, match=match):
        Qwen3Config.from_dict(raw)


def test_registry():
    assert "Qwen3ForCausalLM" in known_architectures() and "qwen3" in known_architectures()
    assert resolve({"architectures": ["Qwen3ForCausalLM"]}) is resolve({"model_type": "qwen3"})
    for raw in ({"architectures": ["Qwen3MoeForCausalLM"], "model_type": "qwen3_moe"}, {"architectures": ["LlamaForCausalLM"], "model_type": "llama"}):
        with pytest.raises(ConfigError, match="not supported"):
            resolve(raw)
    with pytest.raises(ConfigError, match="neither"):
        resolve({})


def test_read_config_json(tmp_path):
    with pytest.raises(ConfigError, match="does not exist"):
        read_config_json(tmp_path)
    (tmp_path / "config.json").write_text("{ not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(QWEN3_0_6B))
    assert read_config_json(tmp_path)["hidden_size"] == 1024
