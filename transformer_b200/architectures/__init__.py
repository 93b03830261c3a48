"""Architectures known to the registry.  Importing this package registers them."""
from . import dumalix, llama, salepel, zufadra  # noqa: F401
