"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step takes portions of prompts beside single decoded tokens, cut anywhere, runs exactly the
tokens it is given as one flat batch and returns the logits at the wanted places. The reference has
three entry points for this (prefill_slot, decode, fused_step: crates/specrt/src/runtime/step.rs:121-232,
crates/specrt/src/runtime/fused.rs:14-61) and allows one prompt portion beside decode rows; here one
function takes any mix.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Hashable, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..parts.decoder import Decoder
from .context import Segment, StepContext, build_context
from .runtime import Runtime


@dataclass
class StepEntry:
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


class ModelRunner:
    """Owns nothing but the wiring: a bound decoder, a cache manager and a runtime."""

    def __init__(self, decoder: Decoder, cache: CacheManager, rt: Runtime):
        self.decoder, self.cache, self.rt = decoder, cache, rt
        self.vocab = decoder.plan.vocab_size

    def step(self, entries: Sequence[StepEntry], check: bool = True, trace: Optional[list] = None) -> Optional[torch.Tensor]:
        """Run one step. Requests must be admitted to the cache manager; every entry continues its
        request where the last step left it. Returns float32 logits [wanted, vocab] on the device in
        the order of the entries and of their `want`, or None when nothing is wanted.
        Raises OutOfPages (and changes nothing) if a request cannot get its pages. `trace`: a list that receives the
        residual stream at the wanted rows after the embedding and after every schedule entry (debugging)."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return None
        self.rt.activate()
        seen = set()
        for e in entries:
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            toks = np.asarray(e.tokens)
            if toks.min() < 0 or toks.max() >= self.vocab:
                bad = int(toks[(toks < 0) | (toks >= self.vocab)][0])
                raise ValueError(f"request {e.request!r}: token id {bad} is outside the vocabulary of {self.vocab}")
        # pages first, all or nothing across the batch
        done = []
        try:
            for e in entries:
                self.cache.extend(e.request, self.cache.length(e.request) + len(e.tokens))
                done.append(e)
        except Exception:
            for e in done:  # give back what this step took: shrink to the committed length
                self.cache.shrink_to_committed(e.request)
            raise
        segments = [Segment(e.request, self.cache.slot(e.request), self.cache.length(e.request), e.tokens, e.want) for e in entries]
        tables = self.cache.step_tables([e.request for e in entries])
        dev_tables = [torch.from_numpy(t).pin_memory().to(self.rt.device, non_blocking=True) for t in tables]
        ctx = build_context(self.rt, segments, self.cache.views(dev_tables))
        ctx.trace = trace
        logits = self.decoder.forward(ctx)
        for e in entries:
            self.cache.commit(e.request, self.cache.length(e.request) + len(e.tokens))
        if check:
            self.rt.check_status()
        return logits
