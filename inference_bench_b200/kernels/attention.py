"""Chooses the attention kernel for a step: tensor-core kernels where a specialisation exists for
the head size and precision, the generic kernel otherwise. All of them read keys and values
through the block table and give the same result up to rounding."""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


def paged_attention(ctx, q: torch.Tensor, cache: ops.KvLayerView, heads: int, window: Optional[int], scale: float) -> torch.Tensor:
    """q [T, heads*hd] (activation dtype) -> attention output of the same shape and dtype."""
    out = ctx.rt.empty(tuple(q.shape), q.dtype)
    ops.attention_generic(q, cache, ctx.positions, ctx.seg_of_token, window, scale, out, heads, ctx.rt.status)
    return out
