"""Architectures that ship with the engine.  Importing this package registers them."""
from . import qwen2  # noqa: F401
