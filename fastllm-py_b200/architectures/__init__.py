"""Importing this package registers the architectures the engine ships with."""
from . import lasonex, llama, tigitar  # noqa: F401
