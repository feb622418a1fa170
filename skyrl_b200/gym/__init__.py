"""Gymnasium-style environments for LLM agents (the counterpart of the ``skyrl_gym`` package)."""

from . import envs  # noqa: F401  (registers the built-in environments)
from .core import Env, EnvStepOutput
from .registration import make, pprint_registry, register, registry

__all__ = ["Env", "EnvStepOutput", "make", "register", "registry", "pprint_registry"]
