"""One-ring sample maps on the icosphere: the 7-tap hexagonal kernels and pooling maps the
icosphere configurations of the benchmark use.

They are thin compositions of the mesh queries in `sphere.Sphere` (the reference's mesh, vertex
for vertex): tap 0 is the vertex itself, taps 1-6 its ring from
get_adjacent_vertex_indices_to_vertices (the 12 valence-5 vertices repeat their first neighbour,
package/ext_modules/src/util/cpp/sphere.cpp:237-238, :665-680).  The vertex domain of a mesh is an
image with H = 1 and W = number of vertices; a map entry is (x = vertex index, y = 0)
(package/layers/util/icosphere_functions.py:259-262).  Because subdivision keeps old vertices at
their indices (sphere.cpp:820-845), the vertices of level L are the first 10 * 4**L + 2 vertices of
level L + 1 and a "level L + 1 -> L" pooling map needs no index translation.
"""
import torch

from .sphere import Sphere


def num_vertices(order):
    return 10 * 4 ** order + 2


def one_ring(order):
    """(V, 6) int64 ring of every vertex of the order-`order` icosphere, in the mesh's walk order."""
    return Sphere.generate_icosphere(order).get_adjacent_vertex_indices_to_vertices()


def _as_map(taps):
    x = taps.float()
    return torch.stack([x, torch.zeros_like(x)], -1).unsqueeze(0).contiguous()


def vertex_kernel_map(order):
    """(1, V, 7, 2) float32 map of the 7-tap one-ring kernel at every vertex of level `order`
    (nearest interpolation)."""
    ring = one_ring(order)
    return _as_map(torch.cat([torch.arange(ring.shape[0]).view(-1, 1), ring], 1))


def pooling_map(order):
    """(1, V_{order-1}, 7, 2) map that pools level `order` down to level `order - 1`: for every
    coarse vertex (the first V_{order-1} fine vertices) itself and its ring in the FINE mesh."""
    nc = num_vertices(order - 1)
    ring = one_ring(order)[:nc]
    return _as_map(torch.cat([torch.arange(nc).view(-1, 1), ring], 1))
