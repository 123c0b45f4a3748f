"""Architectures: each module registers its name, configuration class and builder."""
from . import lopazen, qwen3  # noqa: F401
