"""Importing this package registers every architecture the engine has."""
from . import qwen3  # noqa: F401
