"""Icosphere utilities: mesh generation, sample maps between equirectangular images and mesh
elements, gnomonic kernels at mesh elements.  Names, arguments and results follow the reference's
package/layers/util/icosphere_functions.py; the mesh itself is `sphere.Sphere`.

The vertex (or face) domain of a mesh is treated as an image with H = 1 and W = number of
elements; a map entry is (x = element index, y = 0).
"""
import math

import torch

from ..nn import Resample, Unresample
from . import sphere
from .conversions import (convert_3d_to_spherical, convert_cube_to_3d, convert_spherical_to_image)
from .grids import cube_meshgrid, equirectangular_meshgrid


def generate_icosphere(order=0):
    """Icosphere of the given order (icosphere_functions.py:9-14)."""
    return sphere.Sphere.generate_icosphere(order)


def compute_num_vertices(order):
    """Vertices of an icosphere of the given order, 10 * 4**order + 2 (icosphere_functions.py:20-25)."""
    return 12 * 4 ** order - 6 * sum(4 ** i for i in range(order))


def _element_positions(icosphere, source):
    if source == "face":
        return convert_3d_to_spherical(icosphere.get_face_barycenters())
    if source == "vertex":
        return convert_3d_to_spherical(icosphere.get_vertices())
    raise ValueError("Invalid source ({})".format(source))


# ---- resample maps: (OH, OW, 2) or (OH, OW, P, 2), for Resample / Unresample -----------------------

def image_to_sphere_resample_map(image_shape, icosphere, source="vertex"):
    """(1, V or F, 2): the real-valued pixel (x, y) of an (H, W) equirectangular image that every
    vertex (or face barycentre) of the mesh falls on (icosphere_functions.py:383-405)."""
    return convert_spherical_to_image(_element_positions(icosphere, source), image_shape).view(1, -1, 2)


def faces_to_equirectangular_resample_map(icosphere, image_shape):
    """icosphere_functions.py:271-275."""
    return convert_spherical_to_image(_element_positions(icosphere, "face"), image_shape)


def vertices_to_equirectangular_resample_map(icosphere, image_shape):
    """icosphere_functions.py:281-285."""
    return convert_spherical_to_image(_element_positions(icosphere, "vertex"), image_shape)


def _barycentric_map(samples, order, keepdim, nearest):
    _, V, W = sphere.Sphere.get_planar_conv_operator_from_samples(samples, order, keepdim, nearest)
    V = torch.stack((V, torch.zeros_like(V)), -1)
    return V.float(), W.float()


def sphere_to_samples_resample_map(sample_map, order, nearest=False):
    """Vertices (OH, OW, 3, 2) and barycentric weights (OH, OW, 3) of the face of an order-`order`
    icosphere that every (lon, lat) sample falls in (icosphere_functions.py:352-377)."""
    return _barycentric_map(sample_map, order, False, nearest)


def sphere_to_image_resample_map(order, image_shape, nearest=False):
    """The same for the pixel centres of an equirectangular image (icosphere_functions.py:291-315)."""
    lat, lon, _, _ = equirectangular_meshgrid(image_shape)
    return _barycentric_map(torch.stack((lon, lat), -1).contiguous(), order, False, nearest)


def sphere_to_cube_resample_map(order, cube_dim, nearest=False):
    """The same for the pixels of a cube map (icosphere_functions.py:321-346)."""
    v, u, index = cube_meshgrid(cube_dim)
    samples = convert_3d_to_spherical(convert_cube_to_3d(torch.stack((u, v), -1), index, cube_dim))
    return _barycentric_map(samples.contiguous(), order, False, nearest)


# ---- colour transfer between images and vertices ---------------------------------------------------

def _normalised_scatter(img, sample_map, interp_map, num_vertices, nearest):
    sample_map, interp_map = sample_map.to(img.device), interp_map.to(img.device)
    layer = Resample("nearest" if nearest else "bispherical")
    out = layer(img, sample_map, (1, num_vertices), interp_map)
    total = torch.zeros(out.shape[-1], device=img.device)
    total.index_add_(0, sample_map[..., 0].long().view(-1), interp_map.view(-1))
    return out / (total + 1e-12)


def resample_rgb_to_vertex(img, icosphere, order, nearest=False):
    """Equirectangular image (B, C, H, W) -> per-vertex values (B, C, 1, V): every pixel is spread
    over the three vertices of the face it falls in, then normalised by the weight each vertex
    received (icosphere_functions.py:58-88)."""
    sm, im = sphere_to_image_resample_map(order, img.shape[-2:], nearest)
    return _normalised_scatter(img, sm, im, icosphere.num_vertices(), nearest)


def resample_cube_to_vertex(cube, icosphere, order, nearest=False):
    """Cube-map image -> per-vertex values (icosphere_functions.py:94-124)."""
    sm, im = sphere_to_cube_resample_map(order, cube.shape[-2], nearest)
    return _normalised_scatter(cube, sm, im, icosphere.num_vertices(), nearest)


def resample_vertex_to_rect(vertices, image_shape, order, nearest=False):
    """Per-vertex values (B, C, 1, V) -> equirectangular image by barycentric interpolation
    (icosphere_functions.py:31-52)."""
    sm, im = sphere_to_image_resample_map(order, image_shape, nearest)
    layer = Unresample("nearest" if nearest else "bispherical")
    return layer(vertices, sm.to(vertices.device), im.to(vertices.device))


# ---- kernel maps: (OH, OW, K, 2) or (OH, OW, K, P, 2), for mapped convolutions -----------------------

def gnomonic_kernel(spherical_coords, kh, kw, res_lat, res_lon):
    """(lon, lat) of a kh x kw grid on the tangent plane at every given (N, 2) position, spacing
    (res_lon, res_lat), projected back to the sphere -> (1, N, kh * kw, 2)
    (icosphere_functions.py:135-184)."""
    n = spherical_coords.shape[0]
    lon = spherical_coords[..., 0].reshape(1, n, 1)
    lat = spherical_coords[..., 1].reshape(1, n, 1)
    i = (torch.arange(kh) - kh // 2).double()
    j = (torch.arange(kw) - kw // 2).double()
    y = (i * res_lat).float().view(kh, 1).expand(kh, kw).reshape(1, 1, -1)
    x = (j * res_lon).float().view(1, kw).expand(kh, kw).reshape(1, 1, -1)
    rho = (x ** 2 + y ** 2).sqrt()
    nu = rho.atan()
    out_lat = (nu.cos() * lat.sin() + y * nu.sin() * lat.cos() / rho).asin()
    out_lon = lon + torch.atan2(x * nu.sin(), rho * lat.cos() * nu.cos() - y * lat.sin() * nu.sin())
    centre = torch.zeros(kh * kw, dtype=torch.bool)
    centre[(kh // 2) * kw + kw // 2] = True
    out_lat = torch.where(centre, lat.expand_as(out_lat), out_lat)
    out_lon = torch.where(centre, lon.expand_as(out_lon), out_lon)
    out_lon = ((out_lon + math.pi) % (2 * math.pi)) - math.pi
    return torch.stack((out_lon, out_lat), -1)


def gnomonic_kernel_from_sphere(icosphere, kh, kw, res_lat, res_lon, source="vertex"):
    """Gnomonic kernels centred at every vertex (or face barycentre) of the mesh
    (icosphere_functions.py:190-223)."""
    return gnomonic_kernel(_element_positions(icosphere, source), kh, kw, res_lat, res_lon)


def vertex_to_vertex_kernel_map(icosphere, kh, kw, order, nearest=False):
    """Weighted kernel map for a mapped convolution between meshes: a kh x kw gnomonic kernel at
    every vertex of `icosphere`, each tap expressed through the three vertices of the face of an
    order-`order` icosphere it falls in -> vertices (1, V, kh * kw, 3, 2), barycentric weights
    (1, V, kh * kw, 3) (icosphere_functions.py:229-262)."""
    res = icosphere.get_vertex_resolution()
    samples = gnomonic_kernel_from_sphere(icosphere, kh, kw, res, res, source="vertex")
    return _barycentric_map(samples.contiguous(), order, True, nearest)
