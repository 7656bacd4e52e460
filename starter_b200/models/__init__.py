"""Architectures.  Importing this package registers every architecture it holds."""

from . import kudazen, nazulorn, qwen3  # noqa: F401
