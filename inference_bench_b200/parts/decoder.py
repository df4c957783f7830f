"""The generic decoder: builds every part a `ModelPlan` names and runs the plan's schedule.

It knows no architecture. Layers are built once each; the schedule says which layer runs when and
which cache each execution uses, so a layer may run twice or read another execution's cache.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import base
from .plan import ModelPlan, PartSpec


def _build(table: dict, what: str, spec: PartSpec):
    params = dict(spec.params)
    if isinstance(params.get("position"), PartSpec):
        params["position"] = _build(base.POSITION_ENCODINGS, "position encoding", params["position"])
    return base.make(table, what, spec.kind, **params)


class Decoder:
    def __init__(self, plan: ModelPlan):
        plan.validate()
        self.plan = plan
        self.embedding: base.Embedding = _build(base.EMBEDDINGS, "embedding", plan.embedding)
        self.blocks: list[base.Block] = []
        for lp in plan.layers:
            if lp.block not in base.BLOCKS:
                raise KeyError(f"no block arrangement {lp.block!r} is registered")
            self.blocks.append(base.BLOCKS[lp.block](
                _build(base.NORMS, "norm", lp.mixer_norm), _build(base.MIXERS, "mixer", lp.mixer),
                _build(base.NORMS, "norm", lp.feed_forward_norm), _build(base.FEED_FORWARDS, "feed-forward", lp.feed_forward)))
        self.final_norm: base.Norm = _build(base.NORMS, "norm", plan.final_norm)
        self.head: base.Head = _build(base.HEADS, "head", plan.head)
        self.rt = None

    # ------------------------------------------------------------ what the loader and the cache need
    def parts(self) -> list[base.Part]:
        out: list[base.Part] = [self.embedding]
        for b in self.blocks:
            out += b.parts()
        return out + [self.final_norm, self.head]

    def weight_specs(self) -> list[base.WeightSpec]:
        seen: dict[str, base.WeightSpec] = {}
        for p in self.parts():
            for s in p.weight_specs():
                if s.name in seen and seen[s.name].shape != s.shape:
                    raise ValueError(f"tensor {s.name} is wanted with shapes {seen[s.name].shape} and {s.shape}")
                seen[s.name] = s
        return list(seen.values())

    def cache_needs(self) -> list:
        """Per schedule entry: the need of the execution's own cache, or None when it has none or
        reads another entry's."""
        return [None if e.cache_of is not None else self.blocks[e.layer].mixer.cache_need() for e in self.plan.schedule]

    def cache_sources(self) -> list[int]:
        """Per schedule entry: the entry whose cache it uses (itself when it owns one)."""
        return [i if e.cache_of is None else e.cache_of for i, e in enumerate(self.plan.schedule)]

    def bind(self, weights: dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        for p in self.parts():
            p.bind(weights, rt)

    # ------------------------------------------------------------ one step
    @staticmethod
    def _residual_rows(ctx, x: torch.Tensor, pending: Optional[torch.Tensor]) -> torch.Tensor:
        """The residual stream at the wanted rows as it stands after a block: x plus the contribution the block left
        for the next norm to add. Debugging only (a step with `ctx.trace` set): it copies with torch, off the serving path,
        like the reference's per-layer trace buffer (crates/specrt/src/runtime.rs:1406-1412, 2480-2504)."""
        rows = ctx.logit_rows.long()
        out = x.index_select(0, rows)
        if pending is not None:
            for p in range(pending.shape[0]):
                out = out + pending[p].index_select(0, rows)
        return out

    def forward(self, ctx) -> Optional[torch.Tensor]:
        """Runs the step's tokens through the schedule; returns float32 logits [K, V] at the wanted
        rows, or None when no row is wanted (the caches are still filled)."""
        nvtx = torch.cuda.nvtx if ctx.rt.options.nvtx else None
        if nvtx:
            nvtx.range_push(f"step {ctx.n_tokens} tokens in {ctx.n_segments} segments")
            nvtx.range_push("embedding")
        x = self.embedding.forward(ctx)
        if nvtx:
            nvtx.range_pop()
        pending = None
        trace = ctx.trace
        if trace is not None:
            trace.append(self._residual_rows(ctx, x, None))
        for i, e in enumerate(self.plan.schedule):
            if nvtx:
                nvtx.range_push(f"entry {i} layer {e.layer}")
            pending = self.blocks[e.layer].forward(ctx, x, pending, ctx.caches[i] if ctx.caches else None)
            if nvtx:
                nvtx.range_pop()
            if trace is not None:
                trace.append(self._residual_rows(ctx, x, pending))
        logits = None
        if ctx.logit_rows.shape[0] != 0:
            if nvtx:
                nvtx.range_push("head")
            h = self.final_norm.forward(ctx, x, pending, rows=ctx.logit_rows)
            logits = self.head.forward(ctx, h)
            if nvtx:
                nvtx.range_pop()
        if nvtx:
            nvtx.range_pop()
        return logits
