from . import grid_indexing, grid_sample, indexing, neighbors  # noqa: F401
