"""Architectures: importing this package registers every one of them."""

from . import bunosun, llama, puvirax, rerilorn, simetar  # noqa: F401
