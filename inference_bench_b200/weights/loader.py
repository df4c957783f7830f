"""Loads the tensors a model asks for, by name, and says everything that is wrong at once.

Stored precision is kept: BF16 stays bfloat16, F32 stays float32 (F16 is widened to float32, so no
bit is lost), integer tables become int32. What the runtime's mode needs is decided later by the
parts (`Runtime.matrix`, `Runtime.vector`). The reference names one problem per error
("{name} is not in the checkpoint", "{name} has shape [...], expected [...]":
crates/specrt/src/weights.rs:258-273, 377-401); here one `WeightError` lists all missing and
unexpected tensors and all wrong shapes.
"""
from __future__ import annotations

from typing import Iterable, Optional

import torch

from ..parts.base import WeightSpec
from .safetensors_io import Checkpoint, CheckpointError


class WeightError(ValueError):
    """The checkpoint does not hold exactly the tensors the model reads."""

    def __init__(self, missing, unexpected, wrong_shape, other=()):
        self.missing, self.unexpected, self.wrong_shape, self.other = list(missing), list(unexpected), list(wrong_shape), list(other)
        lines = ["the checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  {name} has shape {list(got)}, expected {list(want)}")
        lines += [f"  {o}" for o in self.other]
        super().__init__("\n".join(lines))


def _as_stored(t: torch.Tensor, role: str) -> torch.Tensor:
    if role == "table":
        return t.to(torch.int32)
    if t.dtype == torch.float16:
        return t.to(torch.float32)
    return t


def load_weights(model_dir, specs: Iterable[WeightSpec], ignored: Iterable[str] = (), device: Optional[torch.device] = None) -> dict[str, torch.Tensor]:
    specs = list(specs)
    ckpt = Checkpoint(model_dir)
    try:
        wanted = {s.name: s for s in specs}
        have = set(ckpt.names())
        missing = sorted(set(wanted) - have)
        unexpected = sorted(have - set(wanted) - set(ignored))
        wrong = [(n, ckpt.tensors[n].shape, wanted[n].shape) for n in sorted(set(wanted) & have) if tuple(ckpt.tensors[n].shape) != tuple(wanted[n].shape)]
        other = []
        for n in sorted(set(wanted) & have):
            dt = ckpt.tensors[n].dtype
            floating = dt in ("BF16", "F16", "F32")
            if wanted[n].role == "table" and dt not in ("I32", "I64"):
                other.append(f"{n} is stored as {dt}, expected an integer table")
            elif wanted[n].role != "table" and not floating:
                other.append(f"{n} is stored as {dt}, expected BF16, F16 or F32 (quantized formats are not read)")
        if missing or unexpected or wrong or other:
            raise WeightError(missing, unexpected, wrong, other)
        out = {}
        for s in specs:
            t = _as_stored(ckpt.read(s.name), s.role)
            out[s.name] = t.to(device) if device is not None else t
        return out
    finally:
        ckpt.close()


__all__ = ["load_weights", "WeightError", "CheckpointError"]
