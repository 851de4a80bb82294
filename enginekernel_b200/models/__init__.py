"""Architectures: each module registers its name, configuration class and builder."""
from . import bolelix, lopazen, musavik, qwen3, susalorn  # noqa: F401
