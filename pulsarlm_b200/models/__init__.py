"""Architectures: importing this package registers every one of them."""

from . import bunosun, llama, rerilorn, simetar  # noqa: F401
