"""Architectures.  Importing this package registers them."""
from . import qwen3, movudra, roritar  # noqa: F401
