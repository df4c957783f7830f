"""The model as data: which parts make up each layer, and in which order layers run.

An architecture's builder turns its typed configuration into a `ModelPlan`; the generic decoder
(`parts/decoder.py`) builds the parts from it through the part registries. The reference keeps the
same split: layer kinds are a data pattern (crates/specrt/src/spec.rs:691-698) and each kind has an
op list chosen by conditions (crates/specrt/src/graph.rs:218-244, 347-365).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered kind and its sizes and constants."""
    kind: str
    params: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerPlan:
    """A block: tensor-name prefix, arrangement and the parts it is made of."""
    prefix: str                     # e.g. "model.layers.3"
    block: str                      # registered arrangement, e.g. "prenorm"
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer. `cache_of` names an earlier entry of the schedule whose cache this
    execution reads instead of writing one of its own; None means it owns a cache."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerPlan, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    ignored_tensors: tuple[str, ...] = ()   # names a checkpoint may carry that the model does not read
    root: str = "model"                     # the prefix the decoder's tensors are named under; the loader probes a checkpoint for its other usual places

    def validate(self) -> None:
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, but the model has {len(self.layers)} layers")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which does not run before it")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which owns none")
