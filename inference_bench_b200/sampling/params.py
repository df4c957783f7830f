"""How a request's next token is chosen. Fields and meanings follow the reference's `Sampling`
(crates/specrt/src/runtime.rs:602-630): temperature 0 is greedy; `seed` and the request's step
number feed the noise; top_k 0, top_p 1 and min_p 0 switch those filters off."""
from __future__ import annotations

import functools
import struct
from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0 < self.top_p <= 1:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if not 0 <= self.min_p < 1:
            raise ValueError(f"min_p must be in [0, 1), got {self.min_p}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0

    def row(self, step: int) -> tuple[int, int, int, int, int, int]:
        """The six 32-bit words the sampling kernel reads for one row
        (crates/specrt/src/runtime/step.rs:76-85): inv_temp bits, seed, step, top_k, top_p bits, min_p bits."""
        a, b, d, e, f = _fixed_words(self)
        step &= 0xFFFFFFFF
        return (a, b, step - (1 << 32) if step >= (1 << 31) else step, d, e, f)


@functools.lru_cache(maxsize=4096)
def _fixed_words(p: SamplingParams) -> tuple[int, int, int, int, int]:
    """The words of a row that do not change from step to step."""
    bits = lambda f: struct.unpack("<i", struct.pack("<f", f))[0]
    wrap = lambda u: struct.unpack("<i", struct.pack("<I", u & 0xFFFFFFFF))[0]
    inv_temp = 0.0 if p.greedy else 1.0 / p.temperature
    return (bits(inv_temp), wrap(p.seed), int(p.top_k), bits(p.top_p), bits(p.min_p))


GREEDY = SamplingParams()
