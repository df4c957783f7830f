"""Picks next tokens on the device from logits rows, one kernel for the whole batch."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def pack(self, params: Sequence[SamplingParams], steps: Sequence[int]) -> torch.Tensor:
        rows = np.asarray([p.row(s) for p, s in zip(params, steps)], dtype=np.int32).reshape(-1, 6)
        return torch.from_numpy(rows).pin_memory().to(self.device, non_blocking=True)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], steps: Sequence[int], status: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits float32 [rows, vocab] -> int32 [rows] on the device. steps[i] is how many tokens
        request i has generated so far: with the seed it decides the noise, so a request's tokens do
        not depend on what else is in the batch. With `status` (the runtime's status word) the result
        has one entry more, the word's value after the step."""
        if logits.shape[0] != len(params):
            raise ValueError(f"{logits.shape[0]} logits rows but {len(params)} sampling parameter sets")
        tokens = torch.empty(logits.shape[0] + (1 if status is not None else 0), dtype=torch.int32, device=self.device)
        ops.sample_rows(logits, self.pack(params, steps), tokens, status)
        return tokens
