"""Drop-in counterparts of the reference's ``cache_hub`` modules on this path."""
from .retroinfer_cache import retroinfer_cache  # noqa: F401,E402
