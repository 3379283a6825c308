from .mesh import AXES, BATCH_AXES, LayoutRefused, Mesh, MeshSpec

__all__ = ["AXES", "BATCH_AXES", "LayoutRefused", "Mesh", "MeshSpec"]
