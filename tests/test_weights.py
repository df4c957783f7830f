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


# ------------------------------------------------------------------------------------------ names, roots, strictness, streaming
class _HostRuntime:
    """Stands for the device-side runtime where a test only needs what `bind` asks of it."""

    def __init__(self):
        from inference_bench_b200.config.runtime_options import RuntimeOptions
        self.device, self.options, self.act_dtype = torch.device("cpu"), RuntimeOptions(), torch.bfloat16
        self.live = self.peak = 0

    def upload(self, t, dtype=None):
        return t if dtype is None or t.dtype == dtype else t.to(dtype)

    def matrix(self, w):
        from inference_bench_b200.engine.runtime import LinearWeights
        return LinearWeights(self.upload(w, self.act_dtype), w.shape[0], w.shape[1])

    def vector(self, w):
        return self.upload(w, torch.float32)


def test_rename_rules_and_the_decoders_other_roots(model_dirs, tmp_path):
    from inference_bench_b200.weights.loader import public_names
    dec = _decoder("B")
    tensors = _all(model_dirs["B"])
    want = load_weights(model_dirs["B"], dec.weight_specs())
    # the decoder saved inside a larger model: both usual places of its root (crates/specrt/src/weights.rs:365-375)
    for alt in ("model.language_model", "language_model.model"):
        moved = {(alt + n[len("model"):] if n.startswith("model.") else n): t for n, t in tensors.items()}
        moved["model.visual.patch_embed.weight"] = torch.zeros(4, 4, dtype=torch.bfloat16)      # something the text model does not read
        write_safetensors(tmp_path / "model.safetensors", moved)
        with pytest.raises(WeightError) as e:
            load_weights(tmp_path, dec.weight_specs())
        assert e.value.unexpected == ["model.visual.patch_embed.weight"] and not e.value.missing      # strict: the extra tensor is an error
        got = load_weights(tmp_path, dec.weight_specs(), strict=False)
        assert set(got) == set(want) and all(torch.equal(got[n], want[n]) for n in want)
    # rename rules: parts of names replaced (crates/specrt/src/weights.rs:226-240)
    odd = {n.replace("model.layers.", "transformer.h.").replace("self_attn", "attn"): t for n, t in tensors.items()}
    write_safetensors(tmp_path / "model.safetensors", odd)
    with pytest.raises(WeightError, match="missing tensors"):
        load_weights(tmp_path, dec.weight_specs())
    got = load_weights(tmp_path, dec.weight_specs(), rules={"transformer.h.": "model.layers.", ".attn.": ".self_attn."})
    assert all(torch.equal(got[n], want[n]) for n in want)
    with pytest.raises(CheckpointError, match="both renamed to"):
        public_names(["a.x", "b.x"], ["c.x"], {"a.": "c.", "b.": "c."})


def test_unexpected_tensors_are_a_note_unless_strict(model_dirs, tmp_path):
    from inference_bench_b200.weights.loader import stream_into
    dec = _decoder("A")
    tensors = _all(model_dirs["A"])
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    write_safetensors(tmp_path / "model.safetensors", tensors)
    said = []
    assert stream_into(dec, _HostRuntime(), tmp_path, say=said.append) == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert len(said) == 1 and "1 tensor(s) of the checkpoint are not read" in said[0]
    with pytest.raises(WeightError, match="unexpected tensors"):
        stream_into(_decoder("A"), _HostRuntime(), tmp_path, strict=True)
    # and a missing tensor still lists the unexpected one beside it: one error says everything
    del tensors["model.norm.weight"]
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightError) as e:
        stream_into(_decoder("A"), _HostRuntime(), tmp_path)
    assert e.value.missing == ["model.norm.weight"] and e.value.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]


def test_weights_are_streamed_part_by_part(model_dirs, monkeypatch):
    """While the model is bound, at most one part's source tensors are alive beside what is already bound; a tied
    embedding is read once and shared by the embedding and the head."""
    from inference_bench_b200.weights import loader
    dec = _decoder("A")   # tied
    reads, alive, most = [], [], [0]
    real = loader.WeightStore.read

    def counting(self, name, device=None):
        t = real(self, name, device)
        reads.append(name)
        alive.append(__import__("weakref").ref(t))
        most[0] = max(most[0], sum(r() is not None for r in alive))
        return t

    monkeypatch.setattr(loader.WeightStore, "read", counting)
    loader.stream_into(dec, _HostRuntime(), model_dirs["A"], say=False)
    assert sorted(reads) == sorted(s.name for s in dec.weight_specs())            # every tensor once, the tied table too
    assert dec.head.w.weight.data_ptr() == dec.embedding.table.weight.data_ptr()
    # bound tensors stay alive where binding keeps the stored tensor itself (bfloat16 matrices that need no fusing): what must
    # not happen is that the q, k, v, gate and up sources of every layer are alive at once
    per_layer_sources = 5
    layers = len(dec.blocks)
    kept = sum(r() is not None for r in alive)
    assert kept <= len(reads) - per_layer_sources * layers
    assert most[0] <= kept + 3


def test_the_reference_checkpoints_header_is_what_the_model_asks_for():
    """The names, stored dtypes and shapes of the published Qwen3-0.6B checkpoint, as the reference recorded them
    (crates/specrt/tests/fixtures/headers/qwen3-0.6b.json; it checks its own plan against them in
    crates/specrt/src/plan.rs:569-633), against what this engine's decoder asks of a loader for that model's config.json."""
    from pathlib import Path
    data = Path(__file__).parent / "data" / "reference"
    header = {name: (dtype, tuple(shape)) for name, dtype, shape in json.loads((data / "qwen3-0.6b.header.json").read_text())}
    _, plan = plan_from_config(json.loads((data / "qwen3-0.6b.config.json").read_text()))
    specs = {s.name: s for s in Decoder(plan).weight_specs()}
    assert plan.ignored_tensors == ("lm_head.weight",)                 # tied: the stored head is not read (crates/specrt/src/weights.rs:1396-1405)
    assert set(header) - set(plan.ignored_tensors) == set(specs)
    for name, s in specs.items():
        assert header[name][1] == tuple(s.shape), name
        assert header[name][0] == "BF16"
    assert sum(s.role == "norm" for s in specs.values()) == 28 * 4 + 1 and len(specs) == 28 * 11 + 2


def test_a_checkpoint_written_by_the_official_writer_loads(tmp_path):
    """crates/specrt/tests/fixtures/tiny-qwen3-sliding: config.json with rope_parameters, layer_types and a window; tensors in
    the official writer's order and header layout. The repo's own reader and the test-side reader agree on every value."""
    from pathlib import Path
    folder = Path(__file__).parent / "data" / "reference" / "tiny-qwen3-sliding"
    cfg, plan = plan_from_config(json.loads((folder / "config.json").read_text()))
    assert cfg.rope_theta == 10000.0 and cfg.head_dim == 64 and cfg.sliding_window == 16
    assert cfg.layer_types == ("sliding_attention", "full_attention", "sliding_attention", "full_attention")
    dec = Decoder(plan)
    w = load_weights(folder, dec.weight_specs(), plan.ignored_tensors)       # strict: nothing missing, unexpected or misshapen
    plain = read_safetensors(folder / "model.safetensors")
    assert set(plain) == set(w) and all(torch.equal(w[n].float(), plain[n]) for n in w)
