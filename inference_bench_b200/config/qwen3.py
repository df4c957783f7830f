"""Typed configuration of the Qwen3 dense decoder, read from its own config.json keys.

Mirrors what v0l/inference-bench reads for this family (crates/specrt/src/spec.rs:958-1003 for
the key set, 1461-1738 for the mapping, 1744-1894 for validation; family flags in
crates/specrt/specs/family-qwen3.toml). No size lives in code: every number below comes from
config.json, and a missing required key is an error that names the key.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any, Mapping, Optional

from . import ConfigError


_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "rms_norm_eps")
_LAYER_TYPES = ("full_attention", "sliding_attention")
_DTYPES = ("bfloat16", "float16", "float32")


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = False
    sliding_window: Optional[int] = None
    layer_types: tuple[str, ...] = field(default_factory=tuple)
    torch_dtype: str = "bfloat16"
    model_type: str = "qwen3"
    architectures: tuple[str, ...] = ("Qwen3ForCausalLM",)

    # ---- derived sizes (crates/specrt/src/spec.rs:2175-2194) ----
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def qkv_rows(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    def window_of(self, layer: int) -> Optional[int]:
        """Keys visible from a query in this layer: None = all earlier keys, W = the last W."""
        return self.sliding_window if self.layer_types[layer] == "sliding_attention" else None

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen3Config":
        c = dict(raw.get("text_config") or raw)  # crates/specrt/src/spec.rs:1465-1470
        for key in _REQUIRED:
            if c.get(key) is None:
                raise ConfigError(f"config.json has no {key}")
        heads = int(c["num_attention_heads"])
        hidden = int(c["hidden_size"])
        layers = int(c["num_hidden_layers"])
        head_dim = c.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"config.json has no head_dim and hidden_size {hidden} is not a multiple of num_attention_heads {heads}")
            head_dim = hidden // heads
        theta = c.get("rope_theta")
        params = c.get("rope_parameters")
        if theta is None and isinstance(params, Mapping):
            theta = params.get("rope_theta")
        if theta is None:
            raise ConfigError("config.json has no rope_theta")
        for key in ("rope_scaling", "rope_parameters"):
            scaling = c.get(key)
            if isinstance(scaling, Mapping):
                kind = scaling.get("rope_type", scaling.get("type", "default"))
                if kind not in (None, "default"):
                    raise ConfigError(f"{key} of type {kind!r} is not supported: this engine has plain RoPE only")
        act = c.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported: the Qwen3 feed-forward is SwiGLU (silu)")
        if c.get("attention_bias", False):
            raise ConfigError("attention_bias=true is not supported: Qwen3 dense has no attention bias")
        types = c.get("layer_types")
        window = c.get("sliding_window")
        if types is None and c.get("use_sliding_window") and window:
            # A config that turns windows on without naming the layers: the layers from max_window_layers on are
            # windowed. (The reference reads such a config as full attention everywhere, crates/specrt/src/spec.rs:1678;
            # this engine has windows, so that would be wrong logits without a word.)
            first = c.get("max_window_layers")
            if first is None:
                raise ConfigError("use_sliding_window is true but config.json has neither layer_types nor max_window_layers")
            types = ["sliding_attention" if i >= int(first) else "full_attention" for i in range(layers)]
        if types is None:
            types = ["full_attention"] * layers
        types = tuple(str(t) for t in types)
        if len(types) != layers:
            raise ConfigError(f"layer_types names {len(types)} layers but num_hidden_layers is {layers}")
        for t in types:
            if t not in _LAYER_TYPES:
                raise ConfigError(f"layer type {t!r} is not supported (known: {', '.join(_LAYER_TYPES)})")
        if "sliding_attention" in types:
            if window is None or int(window) <= 0:
                raise ConfigError("layer_types has sliding_attention but config.json has no positive sliding_window")
            window = int(window)
        else:
            window = None  # crates/specrt/src/spec.rs:1678: the window counts only where a layer is windowed
        dtype = c.get("torch_dtype") or c.get("dtype") or "bfloat16"
        if dtype not in _DTYPES:
            raise ConfigError(f"torch_dtype {dtype!r} is not supported (known: {', '.join(_DTYPES)})")
        cfg = cls(
            vocab_size=int(c["vocab_size"]),
            hidden_size=hidden,
            intermediate_size=int(c["intermediate_size"]),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=int(c.get("num_key_value_heads") or heads),
            head_dim=int(head_dim),
            rms_norm_eps=float(c["rms_norm_eps"]),
            rope_theta=float(theta),
            max_position_embeddings=int(c.get("max_position_embeddings") or 2048),  # crates/specrt/src/engine.rs:10
            tie_word_embeddings=bool(c.get("tie_word_embeddings", False)),  # crates/specrt/src/spec.rs:1668
            hidden_act=act,
            attention_bias=False,
            sliding_window=window,
            layer_types=types,
            torch_dtype=dtype,
            model_type=str(c.get("model_type", "qwen3")),
            architectures=tuple(c.get("architectures") or ("Qwen3ForCausalLM",)),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        """The checks of crates/specrt/src/spec.rs:1744-1894 that apply to this family."""
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"num_attention_heads {self.num_attention_heads} is not a multiple of num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for half-rotation RoPE")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")

    def to_dict(self) -> dict[str, Any]:
        """The config.json that reads back to this configuration."""
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        d["layer_types"] = list(self.layer_types)
        d["use_sliding_window"] = self.sliding_window is not None
        d["rope_scaling"] = None
        return d
