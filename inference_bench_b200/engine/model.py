"""From a model (a folder, a hub id, a TOML model spec, or a raw configuration and a seed) to a
decoder bound to a runtime."""
from __future__ import annotations

from typing import Any, Mapping

from .. import models  # noqa: F401  (fills the architecture registry)
from ..config.spec import ModelSpec, resolve_model
from ..parts.decoder import Decoder
from ..registry import resolve
from ..weights.loader import stream_into
from ..weights.random_init import random_tensor
from .runtime import Runtime


def plan_from_config(raw_config: Mapping[str, Any]):
    arch = resolve(raw_config)
    cfg = arch.config_from_dict(raw_config)
    return cfg, arch.plan(cfg)


def load_model(model, rt: Runtime) -> tuple[Any, Decoder]:
    """The configuration chooses the model class; the checkpoint gives the tensors by name, one part
    at a time. `model` is whatever `config.spec.resolve_model` takes."""
    spec: ModelSpec = resolve_model(model)
    if spec.model_dir is None:
        raise FileNotFoundError(f"no weights were found for {spec.name} ({spec.source}): a folder with model.safetensors is needed, or random weights")
    cfg, plan = plan_from_config(spec.raw_config)
    decoder = Decoder(plan)
    decoder.unread_tensors = stream_into(decoder, rt, spec.model_dir, spec.tensors, strict=rt.options.strict_weights)
    return cfg, decoder


def random_model(raw_config: Mapping[str, Any], seed: int, rt: Runtime) -> tuple[Any, Decoder]:
    """A model with random tensors of the kind `write_random_model` stores (the same distributions, seeded per
    tensor name; not the same values: the device's generator is not the host's), made on the device part by part."""
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
