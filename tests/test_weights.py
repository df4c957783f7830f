"""Loading by tensor name, the one error that lists everything wrong, and the random-weights mode (no GPU)."""
import json
import shutil

import pytest
import torch

from inference_bench_b200.engine.model import plan_from_config
from inference_bench_b200.parts.decoder import Decoder
from inference_bench_b200.weights.loader import WeightError, load_weights
from inference_bench_b200.weights.random_init import write_random_model
from inference_bench_b200.weights.safetensors_io import Checkpoint, CheckpointError, write_safetensors
from plain_qwen3 import read_safetensors
from tiny_configs import CONFIGS


def _decoder(name):
    _, plan = plan_from_config(CONFIGS[name]["config"])
    return Decoder(plan)


def _all(folder):
    ck = Checkpoint(folder)
    out = {n: ck.read(n) for n in ck.names()}
    ck.close()
    return out


def test_round_trip_and_precision_kept(model_dirs, tmp_path):
    dec = _decoder("B")
    w = load_weights(model_dirs["B"], dec.weight_specs(), dec.plan.ignored_tensors)
    assert set(w) == {s.name for s in dec.weight_specs()}
    assert all(t.dtype == torch.bfloat16 for t in w.values())
    # the test-side reader sees the same values
    plain = read_safetensors(model_dirs["B"] / "model.safetensors")
    for n, t in w.items():
        assert torch.equal(t.float(), plain[n])
    # a tensor stored in 32-bit stays 32-bit, float16 is widened, bfloat16 stays
    tensors = _all(model_dirs["B"])
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float() + 1e-4
    tensors["model.layers.0.mlp.up_proj.weight"] = tensors["model.layers.0.mlp.up_proj.weight"].to(torch.float16)
    shutil.copy(model_dirs["B"] / "config.json", tmp_path / "config.json")
    write_safetensors(tmp_path / "model.safetensors", tensors)
    w2 = load_weights(tmp_path, dec.weight_specs())
    assert w2["model.norm.weight"].dtype == torch.float32 and torch.equal(w2["model.norm.weight"], tensors["model.norm.weight"])
    assert w2["model.layers.0.mlp.up_proj.weight"].dtype == torch.float32
    assert w2["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(model_dirs, tmp_path):
    dec = _decoder("A")
    tensors = _all(model_dirs["A"])
    del tensors["model.layers.1.self_attn.k_norm.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64, dtype=torch.bfloat16)
    tensors["model.layers.0.mlp.gate_proj.weight"] = torch.zeros(100, 64, dtype=torch.bfloat16)
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 192, dtype=torch.int32)
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightError) as e:
        load_weights(tmp_path, dec.weight_specs(), dec.plan.ignored_tensors)
    err = e.value
    assert err.missing == ["model.layers.1.self_attn.k_norm.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert err.wrong_shape == [("model.layers.0.mlp.gate_proj.weight", (100, 64), (192, 64))]
    text = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "has shape [100, 64], expected [192, 64]", "stored as I32"):
        assert piece in text


def test_tied_model_ignores_a_stored_head(model_dirs, tmp_path):
    dec = _decoder("A")   # tied
    tensors = _all(model_dirs["A"])
    tensors["lm_head.weight"] = torch.ones(256, 64, dtype=torch.bfloat16)
    write_safetensors(tmp_path / "model.safetensors", tensors)
    w = load_weights(tmp_path, dec.weight_specs(), dec.plan.ignored_tensors)
    assert "lm_head.weight" not in w
    with pytest.raises(WeightError, match="unexpected"):
        load_weights(tmp_path, dec.weight_specs())


def test_sharded_checkpoint_and_container_errors(model_dirs, tmp_path):
    dec = _decoder("B")
    tensors = _all(model_dirs["B"])
    names = sorted(tensors)
    half = len(names) // 2
    parts = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    for f, ns in parts.items():
        write_safetensors(tmp_path / f, {n: tensors[n] for n in ns})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {n: f for f, ns in parts.items() for n in ns}}))
    w = load_weights(tmp_path, dec.weight_specs())
    assert all(torch.equal(w[n], tensors[n]) for n in names)
    # the same tensor in two shards
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {n: tensors[n] for n in names[half - 1:]})
    with pytest.raises(CheckpointError, match="appears in both"):
        Checkpoint(tmp_path)
    # a shard the index names but that is missing, no weights at all, a truncated file
    (tmp_path / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(CheckpointError, match="does not exist"):
        Checkpoint(tmp_path)
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(CheckpointError, match="neither"):
        Checkpoint(empty)
    (empty / "model.safetensors").write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00{}")
    with pytest.raises(CheckpointError, match="header length"):
        Checkpoint(empty)


def test_random_weights_mode(tmp_path):
    raw = CONFIGS["B"]["config"]
    a = write_random_model(raw, 7, tmp_path / "a")
    b = write_random_model(raw, 7, tmp_path / "b")
    c = write_random_model(raw, 8, tmp_path / "c")
    assert (a / "config.json").is_file() and (a / "model.safetensors").is_file()
    assert json.loads((a / "config.json").read_text())["hidden_size"] == 96
    ta, tb, tc = _all(a), _all(b), _all(c)
    assert set(ta) == {s.name for s in _decoder("B").weight_specs()}
    assert all(torch.equal(ta[n], tb[n]) for n in ta) and any(not torch.equal(ta[n], tc[n]) for n in ta)
    emb = ta["model.embed_tokens.weight"].float()
    assert abs(emb.std().item() - 0.02) < 0.002 and abs(emb.mean().item()) < 0.002       # N(0, 0.02)
    norm = ta["model.layers.0.input_layernorm.weight"].float()
    assert 0.89 <= norm.min() and norm.max() <= 1.11 and norm.std() > 0.03              # 1 + U(-0.1, 0.1)
    assert all(t.dtype == torch.bfloat16 for t in ta.values())
