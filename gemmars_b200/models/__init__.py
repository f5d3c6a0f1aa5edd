"""Architectures.  Importing this package registers each of them under its config.json names."""
from . import dalerax, kuporax, nogosun, qwen3, toretar  # noqa: F401
