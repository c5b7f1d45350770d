"""Process-group bootstrap, device meshes and the symmetric heap (GPU) with its CPU twin."""
from .context import DistContext, init_context  # noqa: F401
from .mesh import Mesh2D, factor_two_level  # noqa: F401
