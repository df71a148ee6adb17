"""Coordinate conversions between spherical coordinates, unit vectors, equirectangular pixels
and cube-map faces (pure torch; they prepare sample maps and run on whatever device their input
is on).  Same conventions and arithmetic as the reference's package/layers/util/conversions.py:

* spherical pairs are (lon, lat) in radians; lon = atan2(x, z), lat = atan2(-y, hypot(x, z))
  (the y axis points down);
* equirectangular pixels: x = (W / 2)(lon / pi + 1), y = ((H - 1) / 2)(1 - 2 lat / pi);
* cube faces are numbered [-z, -x, +z, +x, +y, -y] and laid out side by side in a
  (cube_dim, 6 * cube_dim) image; pixel centres sit at (u + 0.5, v + 0.5).
"""
import math

import torch


def convert_spherical_to_image(rad, shape):
    """(..., 2) (lon, lat) -> (..., 2) (x, y) pixel coordinates of an (H, W) equirectangular image
    (conversions.py:6-16)."""
    H, W = shape
    x = (W / 2) * (rad[..., 0] / math.pi + 1)
    y = ((H - 1) / 2) * (-2 * rad[..., 1] / math.pi + 1)
    return torch.stack((x, y), -1)


def convert_3d_to_spherical(xyz):
    """(..., 3) -> (..., 2) (lon, lat) (conversions.py:19-29)."""
    x, y, z = xyz[..., 0], xyz[..., 1], xyz[..., 2]
    lat = torch.atan2(-y, (x ** 2 + z ** 2).sqrt())
    lon = torch.atan2(x, z)
    return torch.stack((lon, lat), -1)


def convert_spherical_to_3d(lonlat):
    """(..., 2) (lon, lat) -> (..., 3) unit vectors (conversions.py:32-40)."""
    lon, lat = lonlat[..., 0], lonlat[..., 1]
    return torch.stack((lat.cos() * lon.sin(), -lat.sin(), lat.cos() * lon.cos()), -1)


# (face index, axis whose magnitude dominates, sign of that axis, u numerator, v numerator)
# in the order in which the reference assigns the faces: a later face overwrites an earlier one
# where two magnitudes tie (conversions.py:64-114)
def _cube_faces(x, y, z):
    return ((3, 0, True, -z, -y), (1, 0, False, z, -y), (4, 1, True, x, z), (5, 1, False, x, -z),
            (2, 2, True, x, -y), (0, 2, False, -x, -y))


def convert_3d_to_cube(xyz, cube_dim):
    """(..., 3) -> ((..., 2) (u, v) in face pixels, (..., 1) int64 face index)
    (conversions.py:43-119)."""
    x, y, z = xyz[..., 0], xyz[..., 1], xyz[..., 2]
    mag = (x.abs(), y.abs(), z.abs())
    pos = (x > 0, y > 0, z > 0)
    u = torch.zeros(xyz.shape[:-1], dtype=torch.float32, device=xyz.device)
    v = torch.zeros_like(u)
    index = torch.zeros(xyz.shape[:-1], dtype=torch.int64, device=xyz.device)
    for face, axis, positive, un, vn in _cube_faces(x, y, z):
        others = [a for a in range(3) if a != axis]
        on = (pos[axis] if positive else ~pos[axis]) & (mag[axis] >= mag[others[0]]) & \
             (mag[axis] >= mag[others[1]])
        u = torch.where(on, (0.5 * (un / mag[axis] + 1)).float(), u)
        v = torch.where(on, (0.5 * (vn / mag[axis] + 1)).float(), v)
        index = torch.where(on, torch.full_like(index, face), index)
    uv = torch.stack((u, v), -1) * cube_dim
    return uv, index.unsqueeze(-1)


def convert_spherical_to_cube(lonlat, cube_dim):
    """conversions.py:122-126."""
    return convert_3d_to_cube(convert_spherical_to_3d(lonlat), cube_dim)


def convert_cube_to_3d(uv, index, cube_dim):
    """(..., 2) face pixels + face index (same leading shape, a trailing 1 is accepted) ->
    (..., 3) points on the cube (conversions.py:129-190)."""
    uv = 2 * ((uv.float() + 0.5) / cube_dim) - 1
    u, v = uv[..., 0], uv[..., 1]
    if index.dim() == uv.dim() and index.shape[-1] == 1:
        index = index[..., 0]
    one = torch.ones_like(u)
    # per face: (x, y, z)
    table = {3: (one, -v, -u), 1: (-one, -v, u), 4: (u, one, v), 5: (u, -one, -v),
             2: (u, -v, one), 0: (-u, -v, -one)}
    xyz = torch.zeros(uv.shape[:-1] + (3,), dtype=torch.float32, device=uv.device)
    for face, comps in table.items():
        on = (index == face).unsqueeze(-1)
        xyz = torch.where(on, torch.stack(comps, -1), xyz)
    return xyz


def convert_cubemap_tuple_to_image(uv, idx, cube_dim):
    """(u, v) on face idx -> (x, y) on the (cube_dim, 6 cube_dim) cube-map image
    (conversions.py:193-200)."""
    return torch.stack((idx[..., 0].float() * cube_dim + uv[..., 0], uv[..., 1]), -1)
