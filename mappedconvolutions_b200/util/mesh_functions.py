"""Face / vertex helpers on an icosphere (counterparts of the reference's
package/layers/util/mesh_functions.py)."""
import torch

from ..nn import Unresample
from .conversions import convert_3d_to_spherical, convert_spherical_to_image


def get_downsample_map(hi_res_sphere, low_res_order):
    """Sample map that pools the faces of `hi_res_sphere` down to order `low_res_order`: the four
    children of coarse face f are the fine faces 4 f .. 4 f + 3, so the map lists, per coarse face,
    the spherical positions of its children's barycentres (mesh_functions.py:22-31).
    -> (20 * 4**low_res_order, 4, 2)."""
    op = torch.arange(20 * 4 ** (low_res_order + 1)).view(-1, 4)
    lonlat = convert_3d_to_spherical(hi_res_sphere.get_face_barycenters())
    samples = lonlat[op]
    return convert_spherical_to_image(samples, samples.shape[:2])


def _mean_of_listed(values, index_table, divisor):
    """values (B, C, 1, N), index_table (M, L) -> (B, C, 1, M): sum over the L listed elements of
    values / divisor, as an Unresample with L interpolation points of weight 1 / divisor."""
    idx = index_table.to(values.device).float()
    sample_map = torch.stack((idx, torch.zeros_like(idx)), -1).unsqueeze(0)
    weights = torch.ones(sample_map.shape[:-1], device=values.device) / divisor
    return Unresample("nearest")(values, sample_map, weights)


def vertices_to_faces(vertices, face_vertex_indices):
    """vertices (B, C, 1, V), face_vertex_indices (F, 3) -> (B, C, 1, F): the mean of every face's
    three vertices (mesh_functions.py:34-48)."""
    return _mean_of_listed(vertices, face_vertex_indices, 3)


def faces_to_vertices(faces, adj_face_indices):
    """faces (B, C, 1, F), adj_face_indices (V, 6) -> (B, C, 1, V): the mean of the six faces around
    every vertex (mesh_functions.py:51-65: six weights of 1/3, halved)."""
    return _mean_of_listed(faces, adj_face_indices, 3) / 2
