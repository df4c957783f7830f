"""What one step looks like to the parts: the tokens of the batch and where each one lives.

A batch is a list of segments; a segment is a run of consecutive tokens of one request, starting
at position `pos0` (a decoded token is a segment of length 1). All tokens of all segments form one
flat batch of T rows. The reference's row records are `DecodeRow{slot, token, pos}` and
`PrefillPart{slot, tokens, start}` (crates/specrt/src/runtime/step.rs:23-29,
crates/specrt/src/runtime/fused.rs:6-11); here any number of either may share a step.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Sequence

import numpy as np
import torch

from .runtime import Runtime


@dataclass
class Segment:
    request: Any          # the request's id
    slot: int             # its state slot
    pos0: int             # position of its first token in this step
    tokens: Sequence[int]
    want: Sequence[int] = ()   # places among `tokens` whose logits are wanted


@dataclass
class StepContext:
    rt: Runtime
    segments: list[Segment]
    n_tokens: int
    # host copies (numpy int32)
    h_token_ids: np.ndarray
    h_positions: np.ndarray
    h_seg_of_token: np.ndarray
    h_seg_start: np.ndarray      # [S+1] offsets into the flat batch
    h_seg_pos0: np.ndarray       # [S]
    h_seg_slot: np.ndarray       # [S]
    h_logit_rows: np.ndarray     # [K] flat row index of every wanted place, in entry order
    # device copies (int32)
    token_ids: torch.Tensor
    positions: torch.Tensor
    seg_of_token: torch.Tensor
    seg_start: torch.Tensor
    seg_pos0: torch.Tensor
    seg_slot: torch.Tensor
    logit_rows: torch.Tensor
    # per schedule entry: what the cache manager gives that execution (KvLayerView, StateView or None)
    caches: list = field(default_factory=list)
    # parts may keep per-step results here (e.g. rotation tables shared by all layers)
    memo: dict = field(default_factory=dict)
    # True when the step is being captured into (or replayed from) a CUDA graph: launch shapes must
    # then depend on the batch's sizes only, never on the host copies of positions or tables
    fixed_shape: bool = False
    # None, or a list that the decoder fills with the residual stream at the wanted rows: after the embedding, then after
    # every schedule entry (float32 [wanted, hidden] each). Debugging only.
    trace: Optional[list] = None

    @property
    def n_segments(self) -> int:
        return len(self.segments)

    @property
    def max_segment_len(self) -> int:
        return int(np.max(np.diff(self.h_seg_start))) if self.segments else 0


def build_context(rt: Runtime, segments: list[Segment], caches: Optional[list] = None) -> StepContext:
    """Flatten segments into the arrays of a step and copy them to the device in one transfer."""
    S = len(segments)
    lens = [len(s.tokens) for s in segments]
    T = int(sum(lens))
    seg_start = np.zeros(S + 1, dtype=np.int32)
    np.cumsum(lens, out=seg_start[1:])
    token_ids = np.empty(T, dtype=np.int32)
    positions = np.empty(T, dtype=np.int32)
    seg_of_token = np.empty(T, dtype=np.int32)
    rows: list[int] = []
    for i, s in enumerate(segments):
        a, b = int(seg_start[i]), int(seg_start[i + 1])
        token_ids[a:b] = np.asarray(s.tokens, dtype=np.int64)
        positions[a:b] = np.arange(s.pos0, s.pos0 + (b - a), dtype=np.int32)
        seg_of_token[a:b] = i
        for w in s.want:
            if not 0 <= w < b - a:
                raise ValueError(f"request {s.request!r}: wanted place {w} is outside its {b - a} tokens of this step")
            rows.append(a + int(w))
    seg_pos0 = np.asarray([s.pos0 for s in segments], dtype=np.int32)
    seg_slot = np.asarray([s.slot for s in segments], dtype=np.int32)
    logit_rows = np.asarray(rows, dtype=np.int32)
    # one pinned staging buffer, one copy
    parts = [token_ids, positions, seg_of_token, seg_start, seg_pos0, seg_slot, logit_rows]
    sizes = [p.size for p in parts]
    total = int(sum(sizes))
    staging = torch.empty(max(total, 1), dtype=torch.int32).pin_memory()
    flat = staging.numpy()
    o = 0
    for p, n in zip(parts, sizes):
        flat[o:o + n] = p
        o += n
    dev = staging.to(rt.device, non_blocking=True)
    views = []
    o = 0
    for n in sizes:
        views.append(dev[o:o + n])
        o += n
    return StepContext(rt, segments, T, token_ids, positions, seg_of_token, seg_start, seg_pos0, seg_slot, logit_rows,
                       *views, caches=caches or [])
