"""Architectures: each module turns its configuration into a plan and registers itself."""
from . import llama  # noqa: F401
