"""Pixel grids of the image domains sample maps are built on (pure torch).  Counterparts of the
reference's package/layers/util/grids.py."""
import math

import torch


def get_equirectangular_grid_resolution(shape):
    """Angular spacing (res_lat, res_lon) of an (H, W) equirectangular grid (grids.py:5-10)."""
    H, W = shape
    return math.pi / (H - 1), 2 * math.pi / W


def equirectangular_meshgrid(shape):
    """-> (lat (H, W), lon (H, W), res_lat, res_lon) with latitude running from -pi/2 in row 0 to
    +pi/2 and longitude over W points of [-pi, pi) (grids.py:13-20).  The projection-map builders
    use their own grid with the latitude axis reversed (spherical_projections.py)."""
    H, W = shape
    lat = torch.linspace(-math.pi / 2, math.pi / 2, steps=H).view(-1, 1).expand(-1, W)
    lon = torch.linspace(-math.pi, math.pi, steps=W + 1)[:-1].view(1, -1).expand(H, -1)
    return (lat, lon) + get_equirectangular_grid_resolution(shape)


def cube_meshgrid_resolution(cube_dim):
    """Angular spacing of neighbouring pixels of a cube-map face (grids.py:23-25)."""
    return math.pi / (2 * cube_dim)


def cube_meshgrid(cube_dim):
    """-> (v, u, index), each (cube_dim, 6 cube_dim): row, column inside the face, face number
    (grids.py:28-42)."""
    W = 6 * cube_dim
    v = torch.arange(cube_dim).view(-1, 1).expand(-1, W)
    u = torch.arange(cube_dim).repeat(6).view(1, -1).expand(cube_dim, -1)
    index = torch.arange(6).repeat_interleave(cube_dim).float().view(1, -1).expand(cube_dim, -1)
    return v, u.contiguous(), index.contiguous()


def cartesian_meshgrid(shape):
    """-> (y, x) float grids of an (H, W) image (grids.py:45-50)."""
    H, W = shape
    y = torch.arange(H).view(-1, 1).expand(-1, W).float()
    x = torch.arange(W).view(1, -1).expand(H, -1).float()
    return y, x
