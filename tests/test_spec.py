"""Model specs (TOML), typed runtime options and where a model is found (no GPU)."""
import json
from pathlib import Path

import pytest

from inference_bench_b200.config import ConfigError
from inference_bench_b200.config.runtime_options import RuntimeOptions
from inference_bench_b200.config.spec import find_model_dir, parse_spec, resolve_model
from inference_bench_b200.engine.model import plan_from_config
from tiny_configs import CONFIGS

DATA = Path(__file__).parent / "data" / "reference"

# The reference's own spec of the model it publishes numbers for (crates/specrt/specs/qwen3-0.6b.toml), as text.
QWEN3_06B = '''
name = "qwen3-0.6b"
repo = "Qwen/Qwen3-0.6B"
quant = "bf16"
architecture = "Qwen3ForCausalLM"

[dims]
hidden = 1024
intermediate = 3072
vocab = 151936
tie_embeddings = true

[layers]
count = 28
pattern = ["dense"]

[norm]
kind = "rmsnorm"
eps = 1e-6

[attention]
kind = "gqa"
heads = 16
kv_heads = 8
head_dim = 128
qkv_bias = false
qk_norm = true

[rope]
style = "neox"
theta = 1000000.0

[mlp]
activation = "swiglu"
'''


def test_runtime_options_are_typed_and_closed():
    d = RuntimeOptions()
    assert d.graphs and d.pdl and d.fuse and d.prefill_chunk == 2048 and d.page_size == 64 and d.dtype == "bfloat16"
    o = RuntimeOptions.from_mapping({"graphs": False, "prefill_chunk": "auto", "decode_attention": "split", "dtype": "fp32", "kv_gb": 2})
    assert not o.graphs and o.prefill_chunk == "auto" and o.decode_attention == "split" and o.dtype == "float32" and o.kv_gb == 2.0
    assert o.non_default() == {"graphs": False, "prefill_chunk": "auto", "decode_attention": "split", "dtype": "float32", "kv_gb": 2.0}
    assert RuntimeOptions(fuse=False).qkv_epilogue is False and RuntimeOptions(fuse=False).decode_qk is False and RuntimeOptions().swiglu_epilogue
    with pytest.raises(ConfigError, match="unknown option 'grahps'"):
        RuntimeOptions.from_mapping({"grahps": True})
    with pytest.raises(ConfigError, match="graphs must be true or false"):
        RuntimeOptions.from_mapping({"graphs": 1})
    with pytest.raises(ConfigError, match="page_size must be an integer"):
        RuntimeOptions.from_mapping({"page_size": "16"})
    with pytest.raises(ConfigError, match="prefill_attention = 'mma' is not one of"):
        RuntimeOptions.from_mapping({"prefill_attention": "mma"})
    with pytest.raises(ConfigError, match="page_size must be positive"):
        RuntimeOptions(page_size=0)
    # keyword overrides skip None, so an entry point's unset arguments leave a spec's values alone
    assert o.merged(graphs=None, page_size=16).page_size == 16 and o.merged(graphs=None).graphs is False


def test_a_complete_spec_stands_for_a_config_json():
    spec = parse_spec(QWEN3_06B, "qwen3-0.6b.toml")
    assert spec.name == "qwen3-0.6b" and spec.model_dir is None and spec.runtime == RuntimeOptions()
    cfg, plan = plan_from_config(spec.raw_config)
    ref, _ = plan_from_config(json.loads((DATA / "qwen3-0.6b.config.json").read_text()))
    for f in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
              "rms_norm_eps", "rope_theta", "tie_word_embeddings", "layer_types", "sliding_window"):
        assert getattr(cfg, f) == getattr(ref, f), f
    assert cfg.max_position_embeddings == 2048      # not in the spec: the reference's default context (crates/specrt/src/engine.rs:10)
    assert len(plan.layers) == 28


def test_a_spec_is_layered_over_the_folders_config_json(model_dirs, tmp_path):
    folder = model_dirs["B"]
    text = f'name = "b-long"\nrepo = "{folder}"\n[dims]\nmax_positions = 64\n[runtime]\npage_size = 8\ngraphs = false\nprefill_chunk = 3\n[tensors]\n"transformer." = "model."\n'
    (tmp_path / "b.toml").write_text(text)
    spec = resolve_model(tmp_path / "b.toml")
    assert spec.model_dir == folder and spec.raw_config["max_position_embeddings"] == 64
    assert spec.raw_config["hidden_size"] == CONFIGS["B"]["config"]["hidden_size"]          # what the spec leaves out stays
    assert spec.runtime.page_size == 8 and spec.runtime.graphs is False and spec.runtime.prefill_chunk == 3
    assert spec.tensors == {"transformer.": "model."}
    # a repo relative to the spec file
    rel = tmp_path / "specs"
    rel.mkdir()
    (rel / "b.toml").write_text(f'name = "b"\nrepo = "../{folder.name}"\n')
    (tmp_path / folder.name).symlink_to(folder)
    assert resolve_model(rel / "b.toml").model_dir.resolve() == folder.resolve()
    # a layer pattern repeats over the layers, and a window comes with it
    spec = parse_spec(f'name = "w"\nrepo = "{folder}"\n[layers]\npattern = ["sliding", "full"]\nwindow = 12\n', "w.toml")
    cfg, _ = plan_from_config(spec.raw_config)
    assert cfg.layer_types == ("sliding_attention", "full_attention", "sliding_attention") and cfg.sliding_window == 12


@pytest.mark.parametrize("change,message", [
    ('quant = "bf16"', None),
    ('quant = "nvfp4_g16"', "quant = 'nvfp4_g16' is not supported"),
    ("qk_norm = true", None),
    ("qk_norm = false", "qk_norm = False, but architecture Qwen3ForCausalLM has qk_norm = True"),
    ('style = "neox"', None),
    ('style = "interleaved"', "rope_style = 'interleaved', but architecture"),
    ('activation = "swiglu"', None),
    ('activation = "geglu"', "activation = 'geglu', but architecture"),
    ('kind = "rmsnorm"', None),
    ('kind = "layernorm"', "norm = 'layernorm', but architecture"),
    ("qkv_bias = false", None),
    ("qkv_bias = true", "attention_bias=true is not supported"),
    ('pattern = ["dense"]', None),
    ('pattern = ["linear"]', "layer kind 'linear' is not supported"),
])
def test_what_a_spec_claims_is_checked(change, message):
    key = change.split("=")[0].strip()
    lines = [change if line.split("=")[0].strip() == key and (key != "kind" or "rmsnorm" in line) else line for line in QWEN3_06B.splitlines()]
    text = "\n".join(lines)
    if message is None:
        parse_spec(text)
    else:
        with pytest.raises(ConfigError, match=message):
            plan_from_config(parse_spec(text).raw_config)


def test_spec_errors_name_the_place(tmp_path):
    with pytest.raises(ConfigError, match="not valid TOML"):
        parse_spec("name = ")
    with pytest.raises(ConfigError, match="unknown entry 'layer'"):
        parse_spec(QWEN3_06B + "\n[layer]\ncount = 3\n")
    with pytest.raises(ConfigError, match=r"\[dims\] has no field 'hiden'"):
        parse_spec(QWEN3_06B.replace("hidden = 1024", "hiden = 1024"))
    with pytest.raises(ConfigError, match=r"\[runtime\]: unknown option 'tile'"):
        parse_spec(QWEN3_06B + '\n[runtime]\ntile = "big"\n')
    with pytest.raises(ConfigError, match="is a family description, not a model spec"):    # crates/specrt/specs/family-qwen3.toml
        parse_spec('name = "qwen3"\nkind = "family"\nextends = "base"\n')
    with pytest.raises(ConfigError, match="names no architecture"):
        parse_spec(QWEN3_06B.replace('architecture = "Qwen3ForCausalLM"\n', ""))
    with pytest.raises(ConfigError, match="does not exist"):
        resolve_model(tmp_path / "none.toml")
    with pytest.raises(ConfigError, match="neither a folder nor a model under"):
        resolve_model("no-such-org/no-such-model")
    with pytest.raises(ConfigError, match="config.json has no rms_norm_eps"):
        plan_from_config(parse_spec(QWEN3_06B.replace("eps = 1e-6\n", "")).raw_config)


def test_a_hub_id_is_found_in_the_hub_cache(model_dirs, tmp_path, monkeypatch):
    """models--ORG--NAME/snapshots/<revision>/ under $HF_HUB_CACHE, then $HF_HOME/hub (crates/specrt/src/weights.rs:112-141)."""
    snap = tmp_path / "hub" / "models--acme--tiny-b" / "snapshots" / "0123abcd"
    snap.parent.mkdir(parents=True)
    snap.symlink_to(model_dirs["B"])
    monkeypatch.setenv("HF_HUB_CACHE", str(tmp_path / "hub"))
    spec = resolve_model("acme/tiny-b")
    assert spec.model_dir == snap and spec.name == "tiny-b" and spec.raw_config["hidden_size"] == 96
    monkeypatch.delenv("HF_HUB_CACHE")
    monkeypatch.setenv("HF_HOME", str(tmp_path))
    assert find_model_dir("acme/tiny-b") == snap
    assert find_model_dir("acme/other") is None
    # a spec whose repo is a hub id
    monkeypatch.setenv("HF_HUB_CACHE", str(tmp_path / "hub"))
    assert parse_spec('name = "x"\nrepo = "acme/tiny-b"\n').model_dir == snap


def test_use_sliding_window_without_layer_types():
    raw = dict(CONFIGS["A"]["config"], use_sliding_window=True, sliding_window=8, max_window_layers=1)
    raw.pop("layer_types", None)
    cfg, _ = plan_from_config(raw)
    assert cfg.layer_types == ("full_attention", "sliding_attention") and cfg.window_of(1) == 8 and cfg.window_of(0) is None
    raw.pop("max_window_layers")
    with pytest.raises(ConfigError, match="neither layer_types nor max_window_layers"):
        plan_from_config(raw)
    raw["use_sliding_window"] = False      # a window that is named but switched off counts for nothing
    assert plan_from_config(raw)[0].sliding_window is None
