"""Architectures known to the registry.  Importing this package registers them."""
from . import llama, salepel, zufadra  # noqa: F401
