"""Multi-GPU plumbing: named meshes over ranks, process groups, FSDP / TP / EP sharding,
symmetric (peer-mapped) memory and the fused compute+collective paths."""
from .mesh import Mesh, create_mesh, current_mesh, set_current_mesh  # noqa: F401
