"""Architectures. Importing this package registers them."""
from . import llama, zurerax  # noqa: F401
