"""Architectures.  Importing the package registers them by their `architectures` name."""
from . import llama  # noqa: F401
