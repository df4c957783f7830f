"""Interfaces of the parts a decoder is assembled from, and the registries that map a part's kind
(a string in the model plan) to its class.

A part knows its own sizes and constants (constructor parameters), the tensors it needs by name
(`weight_specs`), what it wants from the cache manager (`cache_need`, mixers only) and how to run
on a step's tokens (`forward`). No part knows which model it is in, and none reads a model config.

Adding a part means subclassing one of the interfaces below and calling the matching `register_*`
function; the decoder, the loader, the cache manager and the step function find it through the plan.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import TYPE_CHECKING, Callable, Optional

import torch

if TYPE_CHECKING:
    from ..engine.context import StepContext
    from ..engine.runtime import Runtime


# ------------------------------------------------------------------ what a part asks of the loader
@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part reads by name. `role` decides precision on the device and random init:
    "matrix": kept in bfloat16 unless stored in 32-bit; random ~ N(0, std)
    "norm":   per-channel scale used in float32; random 1 + U(-0.1, 0.1)
    "table":  integer table, int32."""
    name: str
    shape: tuple[int, ...]
    role: str = "matrix"
    std: float = 0.02


# ------------------------------------------------------------------ what a mixer asks of the cache
@dataclass(frozen=True)
class PagedKV:
    """Keys and values for every token (or for the last `window` tokens) of a request, in pages."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedState:
    """Per-request state of fixed size, zeroed when a request is admitted."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


CacheNeed = Optional[object]  # PagedKV | FixedState | None


class Part:
    """Common life cycle: construct from sizes -> weight_specs() -> bind(weights, runtime)."""

    prefix: str = ""

    def weight_specs(self) -> list[WeightSpec]:
        return []

    def bind(self, weights: dict[str, torch.Tensor], rt: "Runtime") -> None:
        """Take this part's tensors (device tensors, in their stored precision) and prepare them
        for the runtime's mode (fuse, convert, upload derived tables)."""


class Norm(Part):
    def forward(self, ctx: "StepContext", x: torch.Tensor, delta: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: float32 residual stream [T, H], updated in place by `delta` (float32 [P, T, H] or None);
        returns the normalised rows in the runtime's activation dtype. With `rows` only those
        source rows are produced and x is left as it is."""
        raise NotImplementedError


class PositionEncoding(Part):
    def tables(self, ctx: "StepContext") -> tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        """(cos, sin), float32 [T, rotary_dim/2], for the step's tokens; (None, None) for no rotation."""
        raise NotImplementedError


class Mixer(Part):
    adds_to_residual = False   # True: forward takes `residual=` and may add its contribution there itself

    def cache_need(self) -> CacheNeed:
        return None

    def forward(self, ctx: "StepContext", h: torch.Tensor, cache) -> torch.Tensor:
        """h: normalised activations [T, H]; cache: what the cache manager gave this execution
        (a KvLayerView for PagedKV, a StateView for FixedState, None otherwise).
        Returns the residual contribution, float32 [P, T, H] (P partial sums, added in order).
        A part with `adds_to_residual` is called with `residual=x` (float32 [T, H]) as well: it may
        add its contribution to x in place and return None, or leave x alone and return the partial sums."""
        raise NotImplementedError


class FeedForward(Part):
    adds_to_residual = False   # as for a mixer

    def forward(self, ctx: "StepContext", h: torch.Tensor) -> torch.Tensor:
        """Returns the residual contribution, float32 [P, T, H]."""
        raise NotImplementedError


class Embedding(Part):
    def forward(self, ctx: "StepContext") -> torch.Tensor:
        """Returns the float32 residual stream [T, H] for ctx.token_ids."""
        raise NotImplementedError


class Head(Part):
    def forward(self, ctx: "StepContext", h: torch.Tensor) -> torch.Tensor:
        """h: normalised rows [K, H] -> float32 logits [K, V]."""
        raise NotImplementedError


class Block:
    """An arrangement of norm, mixer and feed-forward around the residual stream."""

    def __init__(self, mixer_norm: Norm, mixer: Mixer, feed_forward_norm: Norm, feed_forward: FeedForward):
        self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward = mixer_norm, mixer, feed_forward_norm, feed_forward

    def parts(self) -> list[Part]:
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, ctx: "StepContext", x: torch.Tensor, pending: Optional[torch.Tensor], cache) -> Optional[torch.Tensor]:
        """Runs the block on x (in place). `pending` is a contribution not yet added to x; the
        return value is the block's own last contribution, left for the next norm to add."""
        raise NotImplementedError


# ------------------------------------------------------------------ registries
MIXERS: dict[str, Callable[..., Mixer]] = {}
FEED_FORWARDS: dict[str, Callable[..., FeedForward]] = {}
NORMS: dict[str, Callable[..., Norm]] = {}
POSITION_ENCODINGS: dict[str, Callable[..., PositionEncoding]] = {}
EMBEDDINGS: dict[str, Callable[..., Embedding]] = {}
HEADS: dict[str, Callable[..., Head]] = {}
BLOCKS: dict[str, Callable[..., Block]] = {}


def _register(table: dict, what: str):
    def register(kind: str, factory=None):
        def put(f):
            table[kind] = f
            return f
        return put(factory) if factory is not None else put
    register.__doc__ = f"Register a {what} under a kind name; usable as a decorator."
    return register


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position_encoding = _register(POSITION_ENCODINGS, "position encoding")
register_embedding = _register(EMBEDDINGS, "embedding")
register_head = _register(HEADS, "head")
register_block = _register(BLOCKS, "block arrangement")


def make(table: dict, what: str, kind: str, **params):
    if kind not in table:
        raise KeyError(f"no {what} of kind {kind!r} is registered (known: {', '.join(sorted(table)) or 'none'})")
    return table[kind](**params)
