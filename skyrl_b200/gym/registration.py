"""Environment registry: ``register(id, entry_point)`` and ``make(id, env_config, extras)``
(reference: skyrl-gym/skyrl_gym/envs/registration.py:33,183,233)."""

from __future__ import annotations

import importlib
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Optional, Union


class RegistrationError(Exception):
    pass


@dataclass
class EnvSpec:
    id: str
    entry_point: Union[str, Callable]
    kwargs: Dict[str, Any] = field(default_factory=dict)

    def make(self, **kwargs):
        return make(self.id, **kwargs)


registry: Dict[str, EnvSpec] = {}


def _load(entry_point: Union[str, Callable]) -> Callable:
    if callable(entry_point):
        return entry_point
    if ":" not in entry_point:
        raise RegistrationError(f"entry point '{entry_point}' must look like 'module.path:ClassName'")
    mod, attr = entry_point.split(":", 1)
    return getattr(importlib.import_module(mod), attr)


def register(id: str, entry_point: Union[str, Callable], kwargs: Optional[Dict[str, Any]] = None,
             override: bool = False) -> None:
    if id in registry and not override:
        raise RegistrationError(f"environment '{id}' is already registered")
    registry[id] = EnvSpec(id, entry_point, dict(kwargs or {}))


def make(id: Union[str, EnvSpec], **kwargs):
    """Instantiate an environment; ``kwargs`` (typically ``env_config`` and ``extras``) go to its constructor."""
    spec = id if isinstance(id, EnvSpec) else registry.get(id)
    if spec is None:
        raise RegistrationError(f"no registered environment with id '{id}'; available: {sorted(registry)}")
    ctor = _load(spec.entry_point)
    merged = dict(spec.kwargs)
    merged.update(kwargs)
    return ctor(**merged)


def pprint_registry() -> str:
    return "\n".join(f"{k}: {v.entry_point}" for k, v in sorted(registry.items()))
