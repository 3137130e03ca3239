"""Drop-in counterparts of the reference's ``cache_hub`` modules on this path."""
from .flash_attn_cache import flash_attn_cache  # noqa: F401,E402
from .retroinfer_cache import retroinfer_cache  # noqa: F401,E402
