"""Architectures.  Importing this package registers every architecture it holds."""

from . import qwen3  # noqa: F401
