"""Architectures this library ships.  Importing the package registers them."""

from . import lonasun, nizazen, qwen2  # noqa: F401  (registration)
