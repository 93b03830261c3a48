"""Architectures known to the registry.  Importing this package registers them."""
from . import dumalix, fugavik, llama, salepel, zufadra  # noqa: F401
