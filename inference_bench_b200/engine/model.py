"""From a model folder (or a raw configuration and a seed) to a decoder bound to a runtime."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Mapping, Optional

import torch

from .. import models  # noqa: F401  (fills the architecture registry)
from ..config.qwen3 import read_config_json
from ..parts.decoder import Decoder
from ..registry import resolve
from ..weights.loader import load_weights
from ..weights.random_init import random_tensor
from .runtime import Runtime


def plan_from_config(raw_config: Mapping[str, Any]):
    arch = resolve(raw_config)
    cfg = arch.config_from_dict(raw_config)
    return cfg, arch.plan(cfg)


def load_model(model_dir, rt: Runtime) -> tuple[Any, Decoder]:
    """config.json chooses the model class; model.safetensors gives the tensors by name."""
    cfg, plan = plan_from_config(read_config_json(model_dir))
    decoder = Decoder(plan)
    weights = load_weights(Path(model_dir), decoder.weight_specs(), plan.ignored_tensors, device=rt.device)
    decoder.bind(weights, rt)
    return cfg, decoder


def random_model(raw_config: Mapping[str, Any], seed: int, rt: Runtime) -> tuple[Any, Decoder]:
    """The same tensors `write_random_model` would store, made on the device without touching the disk."""
    cfg, plan = plan_from_config(raw_config)
    decoder = Decoder(plan)
    specs = {s.name: s for s in decoder.weight_specs()}

    class _Lazy(dict):  # tensors are made when a part asks and dropped after it has bound them
        def __missing__(self, name):
            return random_tensor(specs[name], seed, device=rt.device)

    lazy = _Lazy()
    decoder.rt = rt
    for p in decoder.parts():
        p.bind(lazy, rt)
    return cfg, decoder
