"""Sample-map builders for convolution kernels on equirectangular, cube-map and perspective
images (pure torch: they run on the device of `device=` or on the CPU, once per layer; the hot
path only consumes the maps).  Names, arguments and results follow the reference's
package/layers/util/spherical_projections.py; every map is (OH, OW, kh * kw, 2).

The grid these builders use has latitude running from +pi/2 in row 0 DOWN to -pi/2
(spherical_projections.py:106-114), unlike grids.equirectangular_meshgrid.
"""
import math

import numpy as np
import torch

from .conversions import (convert_3d_to_cube, convert_3d_to_spherical, convert_cube_to_3d,
                          convert_spherical_to_3d, convert_spherical_to_image)
from .grids import cube_meshgrid, cube_meshgrid_resolution


def equirectangular_meshgrid(shape, device=None):
    """-> (lat (H, W), lon (H, W), res_lat, res_lon), latitude from +pi/2 (row 0) to -pi/2."""
    H, W = shape
    lat = torch.linspace(math.pi / 2, -math.pi / 2, steps=H, device=device).view(-1, 1).expand(-1, W)
    lon = torch.linspace(-math.pi, math.pi, steps=W + 1, device=device)[:-1].view(1, -1).expand(H, -1)
    return lat, lon, math.pi / (H - 1), 2 * math.pi / W


def _kernel_offsets(kernel_size, step_y, step_x, device=None, dilation=1):
    """Offsets of a kh x kw kernel around its centre tap, row-major: x (1, 1, K), y (1, 1, K).
    (tap index * dilation) * step is formed in float64 and rounded to float32 once."""
    kh, kw = kernel_size
    i = (torch.arange(kh, device=device) - kh // 2).double()
    j = (torch.arange(kw, device=device) - kw // 2).double()
    y = (i * dilation * step_y).float().view(kh, 1).expand(kh, kw).reshape(1, 1, -1)
    x = (j * dilation * step_x).float().view(1, kw).expand(kh, kw).reshape(1, 1, -1)
    return x, y


def _wrap_longitude(lon):
    return ((lon + math.pi) % (2 * math.pi)) - math.pi


def grid_projection_map(shape, kernel_size, dilation=1, device=None):
    """Plain kh x kw grid in (lon, lat) around every pixel, `dilation` pixels apart
    (spherical_projections.py:38-68).  Returned in spherical coordinates, as the reference does."""
    H, W = shape
    lat, lon, res_lat, res_lon = equirectangular_meshgrid(shape, device)
    x, y = _kernel_offsets(kernel_size, res_lat, res_lon, device, dilation)
    return torch.stack((x + lon.reshape(H, W, 1), y + lat.reshape(H, W, 1)), -1)


def perspective_projection_map(shape, kernel_size, dilation, device=None):
    """The regular kh x kw kernel of an ordinary convolution as a sample map in pixel coordinates
    (spherical_projections.py:71-103)."""
    H, W = shape
    r = torch.arange(H, device=device).view(H, 1, 1).float()
    c = torch.arange(W, device=device).view(1, W, 1).float()
    x, y = _kernel_offsets(kernel_size, 1, 1, device, dilation)
    return torch.stack(((x + c).expand(H, W, -1), (y + r).expand(H, W, -1)), -1)


def reverse_equirectangular_projection_map(shape, kernel_size, device=None):
    """Kernel laid out on the equirectangular grid with its horizontal spacing stretched by
    1 / cos(lat) (spherical_projections.py:117-151); (lon, lat) radians."""
    H, W = shape
    lat, lon, res_lat, res_lon = equirectangular_meshgrid(shape, device)
    x, y = _kernel_offsets(kernel_size, res_lat, res_lon, device)
    out_lat = y + lat.reshape(H, W, 1)
    out_lon = _wrap_longitude(x / out_lat.cos() + lon.reshape(H, W, 1))
    return torch.stack((out_lon, out_lat), -1)


def reverse_gnomonic_projection_map(shape, kernel_size, device=None):
    """For every pixel the (lon, lat) of a kh x kw grid laid out on the plane tangent to the sphere
    at that pixel, one pixel of angular spacing apart, projected back onto the sphere (inverse
    gnomonic projection; spherical_projections.py:154-196)."""
    H, W = shape
    kh, kw = kernel_size
    lat, lon, res_lat, res_lon = equirectangular_meshgrid(shape, device)
    x, y = _kernel_offsets(kernel_size, res_lat, res_lon, device)
    lat, lon = lat.reshape(H, W, 1), lon.reshape(H, W, 1)
    rho = (x ** 2 + y ** 2).sqrt()
    nu = rho.atan()
    out_lat = (nu.cos() * lat.sin() + y * nu.sin() * lat.cos() / rho).asin()
    out_lon = lon + torch.atan2(x * nu.sin(), rho * lat.cos() * nu.cos() - y * lat.sin() * nu.sin())
    # the centre tap (rho = 0) is the pixel itself
    centre = torch.zeros(kh * kw, dtype=torch.bool, device=out_lat.device)
    centre[kh * kw // 2] = True
    out_lat = torch.where(centre, lat.expand_as(out_lat), out_lat)
    out_lon = torch.where(centre, lon.expand_as(out_lon), out_lon)
    return torch.stack((_wrap_longitude(out_lon), out_lat), -1)


def get_projection_map(shape, kernel_size, proj="grid", stride=1, dilation=1, device=None):
    """Sample map (OH, OW, kh * kw, 2) of a kernel on an (H, W) equirectangular image, every
    `stride`-th pixel (spherical_projections.py:12-23).  'gnomonic' and 'equirectangular' come in
    pixel coordinates; any other value gives the plain grid in spherical coordinates, exactly as
    the reference does."""
    if proj == "gnomonic":
        m = reverse_gnomonic_projection_map(shape, kernel_size, device)
        m = convert_spherical_to_image(m, m.shape[:2])
    elif proj == "equirectangular":
        m = reverse_equirectangular_projection_map(shape, kernel_size, device)
        m = convert_spherical_to_image(m, m.shape[:2])
    else:
        m = grid_projection_map(shape, kernel_size, dilation, device)
    return m[::stride, ::stride, ...]


def get_perspective_projection_map(shape, kernel_size, stride=1, dilation=1, device=None):
    """spherical_projections.py:33-35."""
    return perspective_projection_map(shape, kernel_size, dilation, device)[::stride, ::stride, ...]


def reverse_cubemap_projection_map(cube_dim, kernel_size):
    """Kernel offsets added in spherical coordinates around every cube-map pixel
    (spherical_projections.py:258-297)."""
    H, W = cube_dim, 6 * cube_dim
    v, u, idx = cube_meshgrid(cube_dim)
    res = cube_meshgrid_resolution(cube_dim)
    lonlat = convert_3d_to_spherical(convert_cube_to_3d(torch.stack((u, v), -1).float(), idx, cube_dim))
    dx, dy = _kernel_offsets(kernel_size, res, res)
    return torch.stack((lonlat[..., 0].reshape(H, W, 1) + dx, lonlat[..., 1].reshape(H, W, 1) + dy), -1)


def cubemap_idx_to_xy(uv, idx, cube_dim):
    """(u, v) on face idx -> (x, y) on the cube-map image (spherical_projections.py:300-307)."""
    return torch.stack((idx[..., 0].float() * cube_dim + uv[..., 0], uv[..., 1]), -1)


def get_reverse_cube_projection_map(cube_dim, kernel_size, stride=1):
    """spherical_projections.py:26-30."""
    spherical = reverse_cubemap_projection_map(cube_dim, kernel_size)
    uv, idx = convert_3d_to_cube(convert_spherical_to_3d(spherical), cube_dim)
    return cubemap_idx_to_xy(uv, idx, cube_dim)[::stride, ::stride, ...]


def cube_to_3d(depth_cubemap):
    """(1, cube_dim, 6 cube_dim) depth cube map -> (3, cube_dim, 6 cube_dim) points: the unit ray
    of every pixel (faces [-z, -x, +z, +x, +y, -y], grid 2 i / cube_dim - 1) times its depth
    (spherical_projections.py:218-255)."""
    cube_dim = depth_cubemap.shape[1]
    dev = depth_cubemap.device
    g = 2.0 * torch.arange(cube_dim, device=dev).float() / cube_dim - 1.0
    v, u = g.view(-1, 1).expand(cube_dim, cube_dim), g.view(1, -1).expand(cube_dim, cube_dim)
    one = torch.ones_like(u)
    faces = [(-u, v, -one), (-one, v, u), (u, v, one), (one, v, -u), (u, one, -v), (u, -one, v)]
    xyz = torch.cat([torch.stack(f, 0) for f in faces], 2)
    return torch.nn.functional.normalize(xyz, dim=0) * depth_cubemap


def cube_to_rect(cubemap, rect_height, rect_width, interpolation="nearest"):
    """cubemap (C, cube_dim, 6 * cube_dim), faces laid out as [-z, -x, +z, +x, +y, -y], resampled
    to a (C, rect_height, rect_width) equirectangular image on the GPU
    (spherical_projections.py:199-213; the kernel replaces include/util/cuda/cube2rect.cuh)."""
    from ..host import impl
    assert len(cubemap.shape) == 3, "Cubemap must have 3 dimensions"
    assert interpolation in ("nearest", "bilinear"), "Invalid interpolation option"
    return impl.cube2rect(cubemap, rect_height, rect_width, 0 if interpolation == "nearest" else 1)


def perspective_resampling(fov, width, height, theta):
    """(lon, lat) of every pixel of a virtual perspective camera with horizontal field of view
    `fov` degrees, rotated by `theta` degrees about the vertical axis
    (spherical_projections.py:310-325)."""
    f = 0.5 * width / np.tan(0.5 * np.radians(fov))
    x, y = np.meshgrid(np.linspace(0.5, width - 0.5, width), np.linspace(0.5, height - 0.5, height))
    x = (x - 0.5 * width) / f
    y = (y - 0.5 * height) / f
    z = 1 / np.sqrt(x ** 2 + y ** 2 + 1)
    x *= z
    y *= z
    theta = -np.radians(theta)
    x = np.cos(theta) * x - np.sin(theta) * z
    z = np.sin(theta) * x + np.cos(theta) * z
    return convert_3d_to_spherical(torch.from_numpy(np.dstack((x, y, z))))
