"""Architectures.  Importing this package registers them."""

from . import gpt2, luporax, rakalix  # noqa: F401
from .model import Model

__all__ = ["Model"]
