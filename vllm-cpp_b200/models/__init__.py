"""Architectures known to the registry."""
from . import gipinex, lutodra, qwen2, retodra, rolesun  # noqa: F401
