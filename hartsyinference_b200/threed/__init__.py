"""3-D geometry utilities: iso-surface extraction and mesh / point-cloud writers."""
from .marching_cubes import marching_cubes  # noqa: F401
from .writers import write_glb, write_obj, write_ply  # noqa: F401
