"""Icosphere construction and the one-ring sample maps built on it (host-side numpy code that
prepares inputs; not a hot path).

The vertex domain of an icosphere is treated as an image with H = 1 and W = number of vertices, a
map entry being (x = vertex index, y = 0), as in the reference's
package/layers/util/icosphere_functions.py:259-262.  As in the reference's subdivision
(package/ext_modules/src/util/cpp/sphere.cpp:811-912) the vertices of level L are the first
10 * 4**L + 2 vertices of level L + 1 and the edge midpoints are appended after them, so a
"level L+1 -> L" pooling map needs no index translation.  Positions are midpoints pushed to the
unit sphere; the reference additionally smooths the old vertices (Loop subdivision), which moves
them by < 2e-4 and does not change connectivity.
"""
import numpy as np
import torch


def num_vertices(order):
    return 10 * 4 ** order + 2


def _icosahedron():
    t = (1.0 + 5.0 ** 0.5) / 2.0
    v = np.array([[-1, t, 0], [1, t, 0], [-1, -t, 0], [1, -t, 0], [0, -1, t], [0, 1, t],
                  [0, -1, -t], [0, 1, -t], [t, 0, -1], [t, 0, 1], [-t, 0, -1], [-t, 0, 1]],
                 dtype=np.float64)
    v /= np.linalg.norm(v, axis=1, keepdims=True)
    f = np.array([[0, 11, 5], [0, 5, 1], [0, 1, 7], [0, 7, 10], [0, 10, 11], [1, 5, 9], [5, 11, 4],
                  [11, 10, 2], [10, 7, 6], [7, 1, 8], [3, 9, 4], [3, 4, 2], [3, 2, 6], [3, 6, 8],
                  [3, 8, 9], [4, 9, 5], [2, 4, 11], [6, 2, 10], [8, 6, 7], [9, 8, 1]], dtype=np.int64)
    return v, f


def _subdivide(v, f):
    e = np.concatenate([f[:, [0, 1]], f[:, [1, 2]], f[:, [2, 0]]], 0)
    e.sort(axis=1)
    uniq, inv = np.unique(e, axis=0, return_inverse=True)
    inv = inv.reshape(-1)
    mid = v[uniq[:, 0]] + v[uniq[:, 1]]
    mid /= np.linalg.norm(mid, axis=1, keepdims=True)
    nv = len(v)
    n = len(f)
    a, b, c = inv[:n] + nv, inv[n:2 * n] + nv, inv[2 * n:] + nv  # midpoints of 01, 12, 20
    nf = np.concatenate([np.stack([f[:, 0], a, c], 1), np.stack([f[:, 1], b, a], 1),
                         np.stack([f[:, 2], c, b], 1), np.stack([a, b, c], 1)], 0)
    return np.concatenate([v, mid], 0), nf


_CACHE = {}


def generate_icosphere(order):
    """-> (vertices (V, 3) float64 on the unit sphere, faces (F, 3) int64)."""
    if order not in _CACHE:
        v, f = _icosahedron()
        for _ in range(order):
            v, f = _subdivide(v, f)
        _CACHE[order] = (v, f)
    return _CACHE[order]


def one_ring(faces, n_vertices, vertices=None):
    """(V, 6) int64 neighbour table; the 12 valence-5 vertices repeat their first neighbour in
    the last slot (as the reference does, sphere.cpp:237-238).  With `vertices` given the
    neighbours are ordered by angle around the vertex."""
    e = np.concatenate([faces[:, [0, 1]], faces[:, [1, 2]], faces[:, [2, 0]],
                        faces[:, [1, 0]], faces[:, [2, 1]], faces[:, [0, 2]]], 0)
    e = np.unique(e, axis=0)  # sorted by (source, target)
    counts = np.bincount(e[:, 0], minlength=n_vertices)
    assert counts.max() <= 6 and counts.min() >= 5
    start = np.concatenate([[0], np.cumsum(counts)[:-1]])
    slot = np.arange(len(e)) - start[e[:, 0]]
    adj = np.full((n_vertices, 6), -1, dtype=np.int64)
    adj[e[:, 0], slot] = e[:, 1]
    if vertices is not None:
        c = vertices
        ref = np.where(np.abs(c[:, 2:3]) < 0.9, np.array([[0.0, 0.0, 1.0]]), np.array([[1.0, 0.0, 0.0]]))
        t1 = np.cross(c, ref)
        t1 /= np.linalg.norm(t1, axis=1, keepdims=True)
        t2 = np.cross(c, t1)
        nb = vertices[np.where(adj >= 0, adj, 0)] - c[:, None, :]
        ang = np.arctan2((nb * t2[:, None, :]).sum(-1), (nb * t1[:, None, :]).sum(-1))
        ang[adj < 0] = np.inf
        order = np.argsort(ang, axis=1, kind="stable")
        adj = np.take_along_axis(adj, order, 1)
    five = adj[:, 5] < 0
    adj[five, 5] = adj[five, 0]
    return adj


def _as_map(taps):
    x = torch.from_numpy(np.ascontiguousarray(taps)).float()
    return torch.stack([x, torch.zeros_like(x)], -1).unsqueeze(0).contiguous()


def vertex_kernel_map(order):
    """(1, V, 7, 2) float32 map of the 7-tap one-ring kernel at every vertex of level `order`:
    tap 0 the vertex itself, taps 1-6 its ring (nearest interpolation)."""
    v, f = generate_icosphere(order)
    adj = one_ring(f, len(v), v)
    return _as_map(np.concatenate([np.arange(len(v))[:, None], adj], 1))


def pooling_map(order):
    """(1, V_{order-1}, 7, 2) map that pools level `order` down to level `order - 1`: for every
    coarse vertex (the first V_{order-1} fine vertices) itself and its ring in the FINE mesh."""
    v, f = generate_icosphere(order)
    adj = one_ring(f, len(v), v)
    nc = num_vertices(order - 1)
    return _as_map(np.concatenate([np.arange(nc)[:, None], adj[:nc]], 1))


def image_to_sphere_resample_map(image_shape, order):
    """(1, V, 2) float32 pixel coordinates of every vertex in an equirectangular image
    (package/layers/util/icosphere_functions.py:383-405 with conversions.py:6-29: lon = atan2(x, z),
    lat = atan2(-y, hypot(x, z)), x_img = (W/2)(lon/pi + 1), y_img = ((H-1)/2)(1 - 2 lat/pi))."""
    H, W = image_shape
    v, _ = generate_icosphere(order)
    lon = np.arctan2(v[:, 0], v[:, 2])
    lat = np.arctan2(-v[:, 1], np.hypot(v[:, 0], v[:, 2]))
    x = (W / 2) * (lon / np.pi + 1)
    y = ((H - 1) / 2) * (1 - 2 * lat / np.pi)
    return torch.from_numpy(np.stack([x, y], -1)).float().unsqueeze(0).contiguous()
