"""Architectures: each module registers its name, configuration class and builder."""
from . import lopazen, qwen3, susalorn  # noqa: F401
