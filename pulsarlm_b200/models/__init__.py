"""Architectures: importing this package registers every one of them."""

from . import llama  # noqa: F401
