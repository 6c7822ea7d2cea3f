"""Architectures: each module registers its config parser and tensor naming."""
from . import llama  # noqa: F401
