"""Drop-in counterparts of the reference's ``cache_hub`` modules on this path."""
