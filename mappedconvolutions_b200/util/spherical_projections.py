"""Sample-map builders for equirectangular images (host-side torch code that prepares inputs of
the mapped convolution; not a hot path).

Conventions follow the reference's package/layers/util/spherical_projections.py:106-114 and
conversions.py:6-16: rows sample latitude from +pi/2 (row 0) down to -pi/2, columns sample
longitude on W points of [-pi, pi); image coordinates are x = (W/2)(lon/pi + 1),
y = ((H-1)/2)(1 - 2 lat/pi).
"""
import math

import torch


def equirectangular_meshgrid(shape):
    """-> (lat (H,W), lon (H,W), res_lat, res_lon)"""
    H, W = shape
    lat = torch.linspace(math.pi / 2, -math.pi / 2, H).view(H, 1).expand(H, W)
    lon = torch.linspace(-math.pi, math.pi, W + 1)[:-1].view(1, W).expand(H, W)
    return lat, lon, math.pi / (H - 1), 2 * math.pi / W


def convert_spherical_to_image(lonlat, shape):
    """(..., 2) of (lon, lat) radians -> (..., 2) of (x, y) pixel coordinates."""
    H, W = shape
    x = (W / 2) * (lonlat[..., 0] / math.pi + 1)
    y = ((H - 1) / 2) * (1 - 2 * lonlat[..., 1] / math.pi)
    return torch.stack((x, y), -1)


def reverse_gnomonic_projection_map(shape, kernel_size):
    """For every pixel, the (lon, lat) of a kh x kw grid laid out on the plane tangent to the
    sphere at that pixel, one pixel of angular spacing apart, projected back onto the sphere
    (inverse gnomonic projection).  -> (H, W, kh*kw, 2).
    Same construction as the reference's spherical_projections.py:154-196."""
    H, W = shape
    kh, kw = kernel_size
    lat, lon, res_lat, res_lon = equirectangular_meshgrid(shape)
    j = torch.arange(kw, dtype=torch.float32) - kw // 2
    i = torch.arange(kh, dtype=torch.float32) - kh // 2
    ty, tx = torch.meshgrid(i * res_lat, j * res_lon, indexing="ij")  # tangent-plane offsets
    tx, ty = tx.reshape(1, 1, -1), ty.reshape(1, 1, -1)
    lat, lon = lat.unsqueeze(-1), lon.unsqueeze(-1)
    rho = torch.sqrt(tx * tx + ty * ty)
    c = torch.atan(rho)
    safe_rho = torch.where(rho > 0, rho, torch.ones_like(rho))
    out_lat = torch.asin(torch.cos(c) * torch.sin(lat) + ty * torch.sin(c) * torch.cos(lat) / safe_rho)
    out_lon = lon + torch.atan2(tx * torch.sin(c),
                                rho * torch.cos(lat) * torch.cos(c) - ty * torch.sin(lat) * torch.sin(c))
    centre = (rho == 0).expand_as(out_lat)
    out_lat = torch.where(centre, lat.expand_as(out_lat), out_lat)
    out_lon = torch.where(centre, lon.expand_as(out_lon), out_lon)
    out_lon = torch.remainder(out_lon + math.pi, 2 * math.pi) - math.pi
    return torch.stack((out_lon, out_lat), -1)


def get_projection_map(shape, kernel_size, proj="gnomonic", stride=1):
    """Sample map (OH, OW, kh*kw, 2) in pixel coordinates for a spherical mapped convolution on
    an equirectangular image (spherical_projections.py:12-23 of the reference; only the gnomonic
    projection is built here)."""
    if proj != "gnomonic":
        raise NotImplementedError("only the gnomonic projection is implemented")
    m = convert_spherical_to_image(reverse_gnomonic_projection_map(shape, kernel_size), shape)
    return m[::stride, ::stride].contiguous()
