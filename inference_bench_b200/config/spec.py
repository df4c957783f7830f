"""Where a model comes from and how it is to be run: a folder, a hub id, or a TOML model spec.

A model spec is a small TOML file in the reference's layout (crates/specrt/specs/qwen3-0.6b.toml:1-32,
`Spec::load` crates/specrt/src/spec.rs:1346-1358, `resolve_spec` crates/specrt/src/engine.rs:71-88):

    name = "qwen3-0.6b"
    repo = "Qwen/Qwen3-0.6B"        # a folder (absolute, or relative to the spec file) or a hub id
    quant = "bf16"
    [dims]      hidden, intermediate, vocab, tie_embeddings, max_positions
    [layers]    count, pattern = ["dense"], window
    [norm]      kind = "rmsnorm", eps
    [attention] kind = "gqa", heads, kv_heads, head_dim, qkv_bias, qk_norm
    [rope]      style = "neox", theta
    [mlp]       activation = "swiglu"
    [tensors]   "old." = "new."     # substring renames applied to the checkpoint's tensor names
    [runtime]   graphs, pdl, fuse, prefill_chunk, page_size, ...   (config/runtime_options.py)

Here the tables are layered over the config.json of `repo` when that folder is found: a value the
spec gives replaces the one of config.json, and what it leaves out stays. Without a config.json the
spec has to give every size itself (plus `architecture`), which is how a random-weights model is
described. The result is a raw mapping in config.json's own keys: the architecture's typed
configuration class reads it as it reads any config.json, so no size is interpreted twice.

Values that config.json has no key for (`qk_norm`, the norm's kind, the rotation's style, the
activation) are claims about the architecture; they are checked against the traits the architecture
registered and a disagreement is an error, never silently ignored.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping, Optional

from . import ConfigError
from .runtime_options import RuntimeOptions

try:  # Python 3.11+
    import tomllib as _toml
except ModuleNotFoundError:  # pragma: no cover
    _toml = None

INDEX = "model.safetensors.index.json"
SINGLE = "model.safetensors"

# spec table -> {field: config.json key}
_KEYS = {
    "dims": {"hidden": "hidden_size", "intermediate": "intermediate_size", "vocab": "vocab_size", "tie_embeddings": "tie_word_embeddings",
             "max_positions": "max_position_embeddings"},
    "layers": {"count": "num_hidden_layers", "window": "sliding_window"},
    "norm": {"eps": "rms_norm_eps"},
    "attention": {"heads": "num_attention_heads", "kv_heads": "num_key_value_heads", "head_dim": "head_dim", "qkv_bias": "attention_bias"},
    "rope": {"theta": "rope_theta", "scaling": "rope_scaling"},
    "mlp": {},
}
# spec table -> {field: trait name}: values without a config.json key
_CLAIMS = {
    "norm": {"kind": "norm", "unit_offset": "norm_unit_offset"},
    "attention": {"kind": "attention", "qk_norm": "qk_norm"},
    "rope": {"style": "rope_style"},
    "mlp": {"activation": "activation"},
}
_PATTERN = {"dense": "full_attention", "full": "full_attention", "sliding": "sliding_attention"}
_TOP = {"name", "repo", "quant", "architecture", "min_engine", *_KEYS, "tensors", "runtime"}


def read_config_json(model_dir) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist")
    try:
        return json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from e


def hub_dir() -> Path:
    """The hub cache, looked up as the reference does (crates/specrt/src/weights.rs:112-120)."""
    if os.environ.get("HF_HUB_CACHE"):
        return Path(os.environ["HF_HUB_CACHE"])
    if os.environ.get("HF_HOME"):
        return Path(os.environ["HF_HOME"]) / "hub"
    return Path(os.environ.get("HOME") or "/") / ".cache" / "huggingface" / "hub"


def find_model_dir(repo: str, base: Optional[Path] = None, need_weights: bool = False) -> Optional[Path]:
    """A local folder (absolute, relative to `base`, or relative to the working directory), else the
    snapshot of a hub id under the hub cache (crates/specrt/src/weights.rs:125-141). None when nothing
    is found. With `need_weights` a folder counts only if it holds model.safetensors or its index."""
    def good(d: Path) -> bool:
        return d.is_dir() and (not need_weights or (d / SINGLE).is_file() or (d / INDEX).is_file())

    cands = [Path(repo)]
    if base is not None and not Path(repo).is_absolute():
        cands.insert(0, base / repo)
    for c in cands:
        if good(c):
            return c
    snapshots = hub_dir() / ("models--" + repo.replace("/", "--")) / "snapshots"
    if snapshots.is_dir():
        for d in sorted(snapshots.iterdir()):
            if good(d) and ((d / "config.json").is_file() or need_weights):
                return d
    return None


@dataclass(frozen=True)
class ModelSpec:
    """A model resolved to the three things the engine needs: a raw configuration in config.json's
    keys, the folder its weights are read from (None: none were found; random weights only), and
    the options it wants to be run with."""
    name: str
    raw_config: Mapping[str, Any]
    model_dir: Optional[Path]
    tensors: Mapping[str, str] = field(default_factory=dict)       # substring renames for checkpoint names
    runtime: RuntimeOptions = field(default_factory=RuntimeOptions)
    source: str = ""


def _check_claims(raw: Mapping[str, Any], claims: Mapping[str, Any], where: str) -> None:
    from ..registry import resolve
    traits = resolve(raw).traits
    for trait, value in claims.items():
        if trait not in traits:
            if value in (False, None):
                continue
            raise ConfigError(f"{where}: {trait} = {value!r} cannot be honoured: architecture {resolve(raw).name} does not say what it does there")
        if traits[trait] != value:
            raise ConfigError(f"{where}: {trait} = {value!r}, but architecture {resolve(raw).name} has {trait} = {traits[trait]!r}")


def parse_spec(text: str, where: str = "model spec", base: Optional[Path] = None) -> ModelSpec:
    if _toml is None:  # pragma: no cover
        raise ConfigError("reading a TOML model spec needs Python 3.11 or newer (tomllib)")
    try:
        doc = _toml.loads(text)
    except _toml.TOMLDecodeError as e:
        raise ConfigError(f"{where} is not valid TOML: {e}") from e
    if doc.get("kind") in ("family", "kernel"):
        raise ConfigError(f"{where}: {doc.get('name', '?')} is a {doc['kind']} description, not a model spec")   # crates/specrt/src/spec.rs:1352-1356
    for k in doc:
        if k not in _TOP:
            raise ConfigError(f"{where}: unknown entry {k!r} (known: {', '.join(sorted(_TOP))})")
    quant = doc.get("quant", "bf16")
    if quant != "bf16":
        raise ConfigError(f"{where}: quant = {quant!r} is not supported: this engine reads bfloat16, float16 and float32 weights only")
    repo = doc.get("repo")
    model_dir = find_model_dir(str(repo), base) if repo else None
    raw: dict[str, Any] = {}
    if model_dir is not None and (model_dir / "config.json").is_file():
        raw = dict(read_config_json(model_dir))
        if isinstance(raw.get("text_config"), Mapping):   # crates/specrt/src/spec.rs:1465-1470
            outer = raw.get("model_type")
            raw = dict(raw["text_config"], **({"model_type": outer} if outer else {}))
    if doc.get("architecture"):
        raw["architectures"] = [str(doc["architecture"])]
        raw.pop("model_type", None)
    claims: dict[str, Any] = {}
    for table, keys in _KEYS.items():
        t = doc.get(table, {})
        if not isinstance(t, Mapping):
            raise ConfigError(f"{where}: [{table}] must be a table")
        for name, value in t.items():
            if name in keys:
                raw[keys[name]] = value
            elif name in _CLAIMS.get(table, {}):
                claims[_CLAIMS[table][name]] = value
            elif table == "layers" and name == "pattern":
                continue
            else:
                raise ConfigError(f"{where}: [{table}] has no field {name!r} (known: {', '.join(sorted([*keys, *_CLAIMS.get(table, {})]))})")
    pattern = doc.get("layers", {}).get("pattern")
    if pattern is not None:
        if not isinstance(pattern, list) or not pattern:
            raise ConfigError(f"{where}: layers.pattern must be a non-empty list of layer kinds")
        for p in pattern:
            if p not in _PATTERN:
                raise ConfigError(f"{where}: layer kind {p!r} is not supported (known: {', '.join(sorted(_PATTERN))})")
        count = raw.get("num_hidden_layers")
        if not isinstance(count, int) or count <= 0:
            raise ConfigError(f"{where}: layers.pattern needs layers.count (or a config.json with num_hidden_layers)")
        raw["layer_types"] = [_PATTERN[pattern[i % len(pattern)]] for i in range(count)]   # the pattern repeats over the layers
    act = claims.get("activation")
    if act is not None:
        raw["hidden_act"] = {"swiglu": "silu"}.get(act, act)
    if "architectures" not in raw and "model_type" not in raw:
        raise ConfigError(f"{where}: no config.json was found for repo {repo!r} and the spec names no architecture")
    _check_claims(raw, claims, where)
    tensors = doc.get("tensors", {})
    if not isinstance(tensors, Mapping) or not all(isinstance(k, str) and isinstance(v, str) for k, v in tensors.items()):
        raise ConfigError(f"{where}: [tensors] must map name parts to name parts")
    runtime = RuntimeOptions.from_mapping(doc.get("runtime", {}), f"{where} [runtime]")
    weights_dir = model_dir if model_dir is not None and ((model_dir / SINGLE).is_file() or (model_dir / INDEX).is_file()) else None
    return ModelSpec(str(doc.get("name") or (repo or "model")), raw, weights_dir, dict(tensors), runtime, where)


def resolve_model(model, options: Optional[RuntimeOptions] = None) -> ModelSpec:
    """`model`: a path ending in .toml (a model spec), a folder with config.json, a hub id whose
    snapshot lies in the hub cache, or a raw config.json mapping (random weights)."""
    if isinstance(model, ModelSpec):
        return model
    if isinstance(model, Mapping):
        return ModelSpec(str(model.get("_name_or_path") or "config"), dict(model), None, {}, options or RuntimeOptions(), "mapping")
    text = str(model)
    if text.endswith(".toml"):
        path = Path(text)
        if not path.is_file():
            raise ConfigError(f"{path} does not exist")
        spec = parse_spec(path.read_text(), str(path), path.resolve().parent)
        return spec
    found = find_model_dir(text)
    if found is None:
        raise ConfigError(f"{text} is neither a folder nor a model under {hub_dir()}")
    name = text.rstrip("/").rsplit("/", 1)[-1].lower()   # crates/specrt/src/engine.rs:85
    return ModelSpec(name, read_config_json(found), found, {}, options or RuntimeOptions(), str(found))
