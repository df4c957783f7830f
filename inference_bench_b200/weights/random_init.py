"""Random weights from a configuration and a seed.

`write_random_model` writes a model folder (config.json, model.safetensors) that loads like any
checkpoint; `random_weights` makes the same kind of tensors directly on a device for models too
large to be worth a trip through the disk. Matrices and embeddings ~ N(0, std) with std 0.02,
norm scales 1 + U(-0.1, 0.1), stored in bfloat16. Each tensor's stream is seeded from (seed, name),
so the values do not depend on the order tensors are made in. The reference has random weights
only in its fixture scripts (crates/specrt/scripts/tiny_sliding.py:39-51).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Any, Iterable, Mapping, Optional

import torch

from ..parts.base import WeightSpec
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(spec: WeightSpec, seed: int, device="cpu", dtype=torch.bfloat16, std: Optional[float] = None) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, spec.name))
    if spec.role == "norm":
        t = 1.0 + (torch.rand(spec.shape, generator=g, device=device, dtype=torch.float32) * 0.2 - 0.1)
    elif spec.role == "matrix":
        t = torch.randn(spec.shape, generator=g, device=device, dtype=torch.float32) * (spec.std if std is None else std)
    else:
        raise ValueError(f"no random initialisation for tensors of role {spec.role!r} ({spec.name})")
    return t.to(dtype)


def random_weights(specs: Iterable[WeightSpec], seed: int, device="cpu", dtype=torch.bfloat16, std: Optional[float] = None) -> dict[str, torch.Tensor]:
    return {s.name: random_tensor(s, seed, device, dtype, std) for s in specs}


def write_random_model(raw_config: Mapping[str, Any], seed: int, out_dir, dtype=torch.bfloat16, std: Optional[float] = None) -> Path:
    """Write `out_dir/config.json` and `out_dir/model.safetensors` for the architecture that
    `raw_config` names; returns the folder. `std` overrides the standard deviation of matrices."""
    from .. import models  # noqa: F401  (fills the architecture registry)
    from ..parts.decoder import Decoder
    from ..registry import resolve

    arch = resolve(raw_config)
    cfg = arch.config_from_dict(raw_config)
    decoder = Decoder(arch.plan(cfg))
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    full = dict(raw_config)
    full.update(arch.config_to_dict(cfg))
    (out / "config.json").write_text(json.dumps(full, indent=2) + "\n")
    write_safetensors(out / "model.safetensors", random_weights(decoder.weight_specs(), seed, "cpu", dtype, std), {"format": "pt", "seed": str(seed)})
    return out
