"""Architectures known to the registry."""
from . import lutodra, qwen2, retodra, rolesun  # noqa: F401
