"""Typed runtime options: every choice that is not the model's own (which kernels, which fusions,
how the cache and the scheduler are sized), in one frozen object that a `Runtime` carries.

The reference keeps the same kind of thing in the `[runtime]` table of a model spec
(`RuntimeOptions`, crates/specrt/src/spec.rs:148-183: backend, graphs, pdl, fuse, tile,
prefill_chunk, ...; unknown fields are an error). The names it has are kept (`graphs`, `pdl`,
`fuse`, `prefill_chunk`); the others belong to this engine's kernels. Nothing here is global: two
engines in one process may run with different options.
"""
from __future__ import annotations

from dataclasses import dataclass, fields, replace
from typing import Any, Mapping, Optional, Union

from . import ConfigError

_CHOICES = {
    "dtype": ("bfloat16", "float32"),
    "gemm": ("auto", "simt", "tcgen05"),
    "prefill_attention": ("auto", "ws", "tcgen05"),
    "decode_attention": ("auto", "stream", "split"),
}
_ALIASES = {"dtype": {"bf16": "bfloat16", "fp32": "float32"}}


@dataclass(frozen=True)
class RuntimeOptions:
    # ---- precision and the matrix product
    dtype: str = "bfloat16"            # "bfloat16": what serving uses; "float32": every tensor and product in IEEE float32
    gemm: str = "auto"                 # "auto": tcgen05 in bfloat16 where the sizes allow; "simt": the FMA kernel; "tcgen05": refuse sizes it cannot take
    pair_min_tokens: int = 129         # the fused gate/up product runs on the CTA-pair kernel from this many tokens on
    pair_always_tokens: int = 2048     # every product does from here on; between the two a cost model decides
    # ---- launches
    graphs: bool = True                # replay steps of decoded tokens as CUDA graphs
    pdl: bool = True                   # programmatic dependent launch: a kernel's set-up overlaps the tail of the one before
    pipeline: bool = True              # keep decode steps one ahead of the host
    # ---- fusion
    fuse: bool = True                  # master switch: False turns every fused form below off
    fuse_qkv_epilogue: bool = True     # q/k norm, rotation and cache write in the q/k/v projection's epilogue (many tokens, head size 128)
    fuse_decode_qk: bool = True        # the same inside the decode attention kernel (steps of decoded tokens only)
    fuse_decode_max_pairs: int = 128   # ... up to this many (token, kv head) pairs
    fuse_swiglu: bool = True           # SiLU(gate) * up in the gate/up product's epilogue
    # ---- attention kernels
    prefill_attention: str = "auto"    # "ws": warp-specialised tcgen05 kernel fed by TMA; "tcgen05": every thread does everything, cp.async; "auto": ws where TMA can serve the page size
    decode_attention: str = "auto"     # "stream": CTAs that stay, ring filled by TMA; "split": one CTA per slice, cp.async; "auto": stream where TMA can serve the page size
    stream_tiles_per_slice: int = 0    # 0: each token's keys in equal slices; n > 0: slices of n tiles at fixed positions
    split_tiles_per_slice: int = 0     # 0: chosen from the step's sizes; n > 0: fixed
    # ---- cache and scheduler
    page_size: int = 64
    num_pages: Optional[int] = None
    kv_gb: Optional[float] = None
    max_num_seqs: int = 64
    max_batched_tokens: int = 8192
    prefill_chunk: Union[int, str] = 2048   # longest portion of one prompt in a step, or "auto"
    # ---- loading
    strict_weights: bool = False       # an unexpected tensor in the checkpoint is an error instead of a note
    # ---- failure reporting
    wait_limit_ms: int = 2000          # how long a bounded wait inside a kernel may last before it gives up and sets the status word
    nvtx: bool = False                 # NVTX ranges around every step and every schedule entry (for ncu --nvtx-include and timelines); off: no cost

    def __post_init__(self):
        for name, allowed in _CHOICES.items():
            v = getattr(self, name)
            if v not in allowed:
                raise ConfigError(f"runtime option {name} = {v!r} is not one of {', '.join(allowed)}")
        for name in ("pair_min_tokens", "pair_always_tokens", "fuse_decode_max_pairs", "page_size", "max_num_seqs", "max_batched_tokens", "wait_limit_ms"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"runtime option {name} must be positive, got {getattr(self, name)}")
        for name in ("stream_tiles_per_slice", "split_tiles_per_slice"):
            if getattr(self, name) < 0:
                raise ConfigError(f"runtime option {name} must not be negative, got {getattr(self, name)}")
        if self.prefill_chunk != "auto" and (not isinstance(self.prefill_chunk, int) or self.prefill_chunk <= 0):
            raise ConfigError(f"runtime option prefill_chunk must be a positive integer or \"auto\", got {self.prefill_chunk!r}")
        if self.num_pages is not None and self.num_pages <= 0:
            raise ConfigError(f"runtime option num_pages must be positive, got {self.num_pages}")
        if self.kv_gb is not None and not self.kv_gb > 0:
            raise ConfigError(f"runtime option kv_gb must be positive, got {self.kv_gb}")

    # -------------------------------------------------------------- what the fused forms resolve to
    @property
    def qkv_epilogue(self) -> bool:
        return self.fuse and self.fuse_qkv_epilogue

    @property
    def decode_qk(self) -> bool:
        return self.fuse and self.fuse_decode_qk

    @property
    def swiglu_epilogue(self) -> bool:
        return self.fuse and self.fuse_swiglu

    # -------------------------------------------------------------- construction
    @classmethod
    def from_mapping(cls, table: Mapping[str, Any], where: str = "[runtime]") -> "RuntimeOptions":
        """A `[runtime]` table. Unknown names and values of the wrong type are errors that name the field."""
        return cls().merged(table, where)

    def merged(self, table: Optional[Mapping[str, Any]] = None, where: str = "runtime options", **kw) -> "RuntimeOptions":
        """These options with the given fields replaced (None values of keyword arguments are skipped)."""
        new = dict(table or {})
        new.update({k: v for k, v in kw.items() if v is not None})
        known = {f.name: f for f in fields(self)}
        clean = {}
        for name, value in new.items():
            if name not in known:
                raise ConfigError(f"{where}: unknown option {name!r} (known: {', '.join(sorted(known))})")
            clean[name] = _typed(name, value, getattr(type(self)(), name) if name not in ("num_pages", "kv_gb", "prefill_chunk") else None, where)
        return replace(self, **clean)

    def to_dict(self) -> dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in fields(self)}

    def non_default(self) -> dict[str, Any]:
        d = RuntimeOptions()
        return {k: v for k, v in self.to_dict().items() if v != getattr(d, k)}


def _typed(name: str, value: Any, default: Any, where: str) -> Any:
    if name in _ALIASES and isinstance(value, str):
        value = _ALIASES[name].get(value, value)
    if name == "prefill_chunk":
        if value == "auto" or (isinstance(value, int) and not isinstance(value, bool)):
            return value
        raise ConfigError(f"{where}: prefill_chunk must be an integer or \"auto\", got {value!r}")
    if name == "num_pages":
        if value is None or (isinstance(value, int) and not isinstance(value, bool)):
            return value
        raise ConfigError(f"{where}: num_pages must be an integer, got {value!r}")
    if name == "kv_gb":
        if value is None or (isinstance(value, (int, float)) and not isinstance(value, bool)):
            return None if value is None else float(value)
        raise ConfigError(f"{where}: kv_gb must be a number, got {value!r}")
    if isinstance(default, bool):
        if not isinstance(value, bool):
            raise ConfigError(f"{where}: {name} must be true or false, got {value!r}")
    elif isinstance(default, int):
        if not isinstance(value, int) or isinstance(value, bool):
            raise ConfigError(f"{where}: {name} must be an integer, got {value!r}")
    elif isinstance(default, str):
        if not isinstance(value, str):
            raise ConfigError(f"{where}: {name} must be a string, got {value!r}")
    return value
