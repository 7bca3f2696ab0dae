"""Architectures. Importing this package registers them."""
from . import llama, lonorax, zurerax  # noqa: F401
