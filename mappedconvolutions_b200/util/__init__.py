"""Utilities of the layer API: sample-map builders, mesh queries, coordinate conversions, k-NN.
Star-exports the same modules, in the same order, as the reference's
package/layers/util/__init__.py:1-9 (its training-loop and file-IO helpers, network_training.py and
read_write.py, are not part of this library); with that order `equirectangular_meshgrid` is the
one of grids.py, as in the reference."""
from . import icosphere, sphere  # noqa: F401
from .sphere import Sphere  # noqa: F401
from .mesh_functions import *  # noqa: F401,F403
from .icosphere_functions import *  # noqa: F401,F403
from .point_functions import *  # noqa: F401,F403
from .spherical_projections import *  # noqa: F401,F403
from .util import *  # noqa: F401,F403
from .conversions import *  # noqa: F401,F403
from .grids import *  # noqa: F401,F403
from .icosphere import one_ring, pooling_map, vertex_kernel_map  # noqa: F401

__all__ = [_n for _n in dir() if not _n.startswith("_")]
