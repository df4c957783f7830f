"""One registry from an architecture's name to its model: a typed configuration class and a
function that turns a configuration into a `ModelPlan`.

The name is looked up as config.json's `architectures[0]`, then its `model_type`. The reference
resolves a family by `model_type` (crates/specrt/src/family.rs:677-704) and answers an unknown one
with "model_type X is not supported".
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping

from .config import ConfigError
from .parts.plan import ModelPlan


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[Mapping[str, Any]], Any]
    plan: Callable[[Any], ModelPlan]
    config_to_dict: Callable[[Any], dict]
    traits: Mapping[str, Any]     # what the architecture does where config.json has no key for it (checked against a model spec's claims)


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(names, config_from_dict, plan, config_to_dict=None, traits=None) -> Architecture:
    """Register one model under every name it goes by (`architectures` entries and `model_type`).
    `traits` says what the architecture does where config.json has no key (for instance
    {"qk_norm": True, "rope_style": "neox"}); a TOML model spec that claims otherwise is refused."""
    names = [names] if isinstance(names, str) else list(names)
    arch = Architecture(names[0], config_from_dict, plan, config_to_dict or (lambda c: c.to_dict()), dict(traits or {}))
    for n in names:
        _ARCHITECTURES[n] = arch
    return arch


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def resolve(raw_config: Mapping[str, Any]) -> Architecture:
    names = list(raw_config.get("architectures") or [])
    for n in names[:1] + ([raw_config["model_type"]] if raw_config.get("model_type") else []):
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    asked = names[0] if names else raw_config.get("model_type")
    if asked is None:
        raise ConfigError("config.json names neither architectures nor model_type")
    raise ConfigError(f"architecture {asked!r} is not supported (known: {', '.join(known_architectures())})")
