from . import grid_indexing, grid_sample, indexing, neighbors, triplet_cache  # noqa: F401
