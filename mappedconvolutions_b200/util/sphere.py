"""Icosphere mesh with the reference's vertex numbering, connectivity and float32 coordinates.

`Sphere` carries the methods of the reference's `_mapped_convolution_ext._sphere.Sphere`
(package/ext_modules/include/util/cpp/sphere.h:131-169) that its Python utilities call.  The
reference keeps a pointer-linked half-edge structure (src/util/cpp/sphere.cpp:129-201); here the
same mesh lives in flat arrays and every step is a whole-array operation:

* a face is three vertex indices in construction order; half-edge h = 3 f + j runs from vertex j
  of face f to vertex (j + 1) % 3, next(h) stays in the face, pair(h) is the half-edge of the
  neighbouring face with the ends exchanged;
* a vertex remembers the LAST half-edge that leaves it in construction order (the reference
  overwrites the pointer face by face, sphere.cpp:176-178, :793-795), and its ring is walked with
  he -> next(pair(he)) (sphere.cpp:226-241) - this fixes the order of the neighbour tables and of the
  float32 sums in the subdivision step;
* Loop subdivision (sphere.cpp:811-912): old vertices keep their indices and are re-positioned with
  the valence weights, one new vertex per edge is appended in the order in which the half-edges
  first meet the edge, every face becomes four faces (corner a, corner b, corner c, centre), so the
  children of face f are 4 f .. 4 f + 3 and the vertices of level L are the first 10 * 4**L + 2
  vertices of every finer level;
* `generate_icosphere` subdivides the raw icosahedron `order` times and normalises at the end
  (sphere.cpp:512-539).

All coordinate arithmetic is float32 in the reference's order of operations, so vertices come out
bit-identical.
"""
import numpy as np
import torch

_F32 = np.float32


def _base_icosahedron():
    r = _F32((1.0 + np.sqrt(5.0)) / 2.0)
    o, z = _F32(1.0), _F32(0.0)
    pts = np.array([[-o, r, z], [o, r, z], [-o, -r, z], [o, -r, z], [z, -o, r], [z, o, r],
                    [z, -o, -r], [z, o, -r], [r, z, -o], [r, z, o], [-r, z, -o], [-r, z, o]],
                   dtype=_F32)
    faces = np.array([[0, 11, 5], [0, 5, 1], [0, 1, 7], [0, 7, 10], [0, 10, 11], [1, 5, 9],
                      [5, 11, 4], [11, 10, 2], [10, 7, 6], [7, 1, 8], [3, 9, 4], [3, 4, 2],
                      [3, 2, 6], [3, 6, 8], [3, 8, 9], [5, 4, 9], [2, 4, 11], [6, 2, 10],
                      [8, 6, 7], [9, 8, 1]], dtype=np.int64)
    return pts, faces


class _Mesh:
    """Flat half-edge arrays of a closed triangle mesh."""

    def __init__(self, vertices, faces, prev_face=None):
        self.v = np.ascontiguousarray(vertices, dtype=_F32)
        self.f = np.ascontiguousarray(faces, dtype=np.int64)
        self.prev_face = prev_face
        nv, nf = len(self.v), len(self.f)
        self.src = self.f.reshape(-1)                      # source vertex of half-edge h
        self.dst = np.roll(self.f, -1, axis=1).reshape(-1)  # vertex it points to
        h = np.arange(3 * nf)
        self.nxt = 3 * (h // 3) + (h % 3 + 1) % 3
        key = self.src * nv + self.dst
        order = np.argsort(key, kind="stable")
        pos = np.searchsorted(key[order], self.dst * nv + self.src)
        assert (pos < len(order)).all() and (key[order][pos] == self.dst * nv + self.src).all(), \
            "mesh is not closed"
        self.pair = order[pos]
        # last half-edge leaving each vertex, in construction order
        self.vert_he = np.zeros(nv, dtype=np.int64)
        self.vert_he[self.src] = h                         # later assignments win
        self._ring = None

    def ring(self):
        """-> (he (V, 6), count (V,)): the half-edges leaving every vertex in the order of the
        reference's ring walk, -1 beyond the vertex's valence."""
        if self._ring is None:
            nv = len(self.v)
            he = np.full((nv, 6), -1, dtype=np.int64)
            cur = self.vert_he.copy()
            alive = np.ones(nv, dtype=bool)
            count = np.zeros(nv, dtype=np.int64)
            for i in range(6):
                he[alive, i] = cur[alive]
                count += alive
                cur = self.nxt[self.pair[cur]]
                alive &= cur != self.vert_he
            assert not alive.any(), "valence above 6"
            self._ring = (he, count)
        return self._ring

    def subdivide(self):
        he, val = self.ring()
        nv, nf = len(self.v), len(self.f)
        # even vertices: beta * (sum of the ring) + (1 - valence * beta) * position, float32 throughout
        beta = np.where(val > 3, 3.0 / (8.0 * val), np.where(val == 3, 3.0 / 16.0, 1.0 / 8.0)).astype(_F32)
        acc = np.zeros((nv, 3), dtype=_F32)
        for i in range(6):
            on = he[:, i] >= 0
            acc[on] = acc[on] + self.v[self.dst[he[on, i]]]
        acc = acc * beta[:, None]
        keep = (1.0 - (val.astype(_F32) * beta).astype(np.float64)).astype(_F32)
        even = acc + self.v * keep[:, None]
        # odd vertices: one per edge, numbered by the first half-edge that meets the edge
        h = np.arange(3 * nf)
        first = h < self.pair
        a, b = _F32(3.0 / 8.0), _F32(1.0 / 8.0)
        hf, pf = h[first], self.pair[first]
        odd = (self.v[self.dst[hf]] + self.v[self.dst[pf]]) * a + \
              (self.v[self.dst[self.nxt[hf]]] + self.v[self.dst[self.nxt[pf]]]) * b
        edge_vertex = np.empty(3 * nf, dtype=np.int64)
        edge_vertex[hf] = nv + np.arange(len(hf))
        edge_vertex[pf] = edge_vertex[hf]
        # faces: (a, b, c) = the face's vertices in the order of its half-edge walk (the vertex the
        # first half-edge points to comes first), alpha / beta / gamma the new vertices on ab, bc, ca
        va, vb, vc = self.f[:, 1], self.f[:, 2], self.f[:, 0]
        al, be, ga = edge_vertex[3 * np.arange(nf) + 1], edge_vertex[3 * np.arange(nf) + 2], \
            edge_vertex[3 * np.arange(nf)]
        nf4 = np.stack([np.stack([va, al, ga], 1), np.stack([vb, be, al], 1),
                        np.stack([vc, ga, be], 1), np.stack([al, be, ga], 1)], 1).reshape(-1, 3)
        return _Mesh(np.concatenate([even, odd.astype(_F32)], 0), nf4, np.repeat(np.arange(nf), 4))

    def normalized(self):
        v = self.v
        n = np.sqrt(v[:, 0] * v[:, 0] + v[:, 1] * v[:, 1] + v[:, 2] * v[:, 2]).astype(_F32)
        m = _Mesh.__new__(_Mesh)
        m.__dict__.update(self.__dict__)
        m.v = (v / n[:, None]).astype(_F32)
        return m


_LEVELS = {}


def _icosphere_mesh(order):
    if order not in _LEVELS:
        if order == 0:
            pts, faces = _base_icosahedron()
            m = _Mesh(pts, faces)
        else:
            m = _icosphere_mesh_raw(order)
        _LEVELS[order] = m.normalized()
    return _LEVELS[order]


_RAW = {}


def _icosphere_mesh_raw(order):
    """The icosahedron subdivided `order` times, not normalised."""
    if order not in _RAW:
        if order == 0:
            pts, faces = _base_icosahedron()
            _RAW[order] = _Mesh(pts, faces)
        else:
            _RAW[order] = _icosphere_mesh_raw(order - 1).subdivide()
    return _RAW[order]


_PLANAR = {}
_PLANAR_DEVICE = {}


def _planar_hierarchy(order):
    """Levels 0..order of the hierarchy the point location walks: the unit icosahedron, then Loop
    subdivisions of it WITHOUT re-normalisation (sphere.cpp:1163, :1214)."""
    levels = _PLANAR.setdefault("levels", [_icosphere_mesh(0)])
    while len(levels) <= order:
        levels.append(levels[-1].subdivide())
    return levels[:order + 1]


def _planar_device_arrays(order, device):
    key = (str(device), order)
    if key not in _PLANAR_DEVICE:
        arrs = []
        for m in _planar_hierarchy(order):
            arrs.append((torch.from_numpy(m.v.copy()).to(device),
                         torch.from_numpy(np.roll(m.f, -1, axis=1).astype(np.int32)).contiguous().to(device),
                         torch.from_numpy((m.pair // 3).reshape(-1, 3).astype(np.int32)).contiguous().to(device)))
        _PLANAR_DEVICE[key] = arrs
    return _PLANAR_DEVICE[key]


class Sphere:
    """Triangle mesh on the sphere with the query methods of the reference's Sphere class.
    Tensors are returned on the CPU with the reference's dtypes (float32 / int64)."""

    @staticmethod
    def get_planar_conv_operator_from_samples(samples, order, keepdim, nearest, device=None):
        """samples (OH, OW, 2) or (OH, OW, K, 2) of (lon, lat) -> [face (OH, OW[, K]) int64,
        vertices (OH, OW[, K], 3) int64, barycentric weights (OH, OW[, K], 3) float32] of the
        order-`order` icosphere face every sample falls in (sphere.cpp:1116-1270).  The search runs
        on the GPU (mc_sphere_locate); results come back on the samples' device."""
        import ctypes

        from .. import _lib
        if device is None:
            device = samples.device if samples.is_cuda else torch.device("cuda", torch.cuda.current_device()) \
                if torch.cuda.is_available() else None
        if device is None:
            raise RuntimeError("point location on the icosphere is CUDA only: no device available "
                               "(this build has no CPU path)")
        k = 1 if samples.dim() == 3 else samples.shape[2]
        lead = tuple(samples.shape[:2]) + ((k,) if (k > 1 or keepdim) else ())
        with torch.cuda.device(device):
            sd = samples.detach().to(device=device, dtype=torch.float32).contiguous()
            n = sd.numel() // 2
            levels = _planar_device_arrays(int(order), device)
            vp = (ctypes.c_void_p * len(levels))(*[a[0].data_ptr() for a in levels])
            fp = (ctypes.c_void_p * len(levels))(*[a[1].data_ptr() for a in levels])
            ap = (ctypes.c_void_p * len(levels))(*[a[2].data_ptr() for a in levels])
            nf = (ctypes.c_int32 * len(levels))(*[a[1].shape[0] for a in levels])
            face = torch.empty(n, dtype=torch.int64, device=device)
            vert = torch.empty(n, 3, dtype=torch.int64, device=device)
            wts = torch.empty(n, 3, dtype=torch.float32, device=device)
            _lib.check(_lib.lib().mc_sphere_locate(
                sd.data_ptr(), n, int(order), vp, fp, ap, nf, 1 if nearest else 0, face.data_ptr(),
                vert.data_ptr(), wts.data_ptr(), torch.cuda.current_stream().cuda_stream))
        out_dev = samples.device
        return [face.view(lead).to(out_dev), vert.view(lead + (3,)).to(out_dev),
                wts.view(lead + (3,)).to(out_dev)]

    def __init__(self, pts=None, faces=None, _mesh=None):
        if _mesh is None:
            _mesh = _Mesh(torch.as_tensor(pts).detach().cpu().numpy(),
                          torch.as_tensor(faces).detach().cpu().numpy())
        self._m = _mesh

    # sphere.cpp:512-539
    @staticmethod
    def generate_icosphere(order=0):
        return Sphere(_mesh=_icosphere_mesh(int(order)))

    def num_vertices(self):
        return len(self._m.v)

    def num_faces(self):
        return len(self._m.f)

    def get_vertices(self):
        """(V, 3) float32, sphere.cpp:545-557."""
        return torch.from_numpy(self._m.v.copy())

    def _face_walk(self):
        # vertices of every face in the order of its half-edge walk (sphere.cpp:212-224): the walk
        # starts at the half-edge 0 -> 1 and lists the vertex each half-edge points to
        return np.roll(self._m.f, -1, axis=1)

    def get_all_face_vertex_indices(self):
        """(F, 3) int64, sphere.cpp:578-591."""
        return torch.from_numpy(self._face_walk().copy())

    def get_all_face_vertex_coords(self):
        """(F, 3, 3) float32, sphere.cpp:560-575."""
        return torch.from_numpy(self._m.v[self._face_walk()].copy())

    def get_face_barycenters(self):
        """(F, 3) float32: ((p0 + p1) + p2) / 3 in walk order, sphere.cpp:203-210, :594-607."""
        p = self._m.v[self._face_walk()]
        return torch.from_numpy((((p[:, 0] + p[:, 1]) + p[:, 2]) / _F32(3.0)).astype(_F32))

    def get_adjacent_face_indices_to_faces(self):
        """(F, 3) int64: the faces across the three half-edges, sphere.cpp:260-272, :631-644."""
        return torch.from_numpy((self._m.pair // 3).reshape(-1, 3).copy())

    def _ring_table(self, values):
        he, val = self._m.ring()
        out = np.where(he >= 0, values[np.where(he >= 0, he, 0)], -1)
        five = val < 6
        out[five, val[five]] = out[five, 0]   # singular points repeat their first entry
        return torch.from_numpy(out.astype(np.int64))

    def get_adjacent_vertex_indices_to_vertices(self):
        """(V, 6) int64 ring of every vertex; the 12 valence-5 vertices repeat their first
        neighbour in the last slot (sphere.cpp:226-241, :665-680)."""
        return self._ring_table(self._m.dst)

    def get_adjacent_face_indices_to_vertices(self):
        """(V, 6) int64 faces around every vertex (sphere.cpp:243-258, :647-662)."""
        return self._ring_table(np.arange(len(self._m.src)) // 3)

    def get_original_face_indices(self):
        """(F,) int64 parent face of every face (sphere.cpp:727-740); zeros for a mesh that was not
        produced by a subdivision."""
        pf = self._m.prev_face
        return torch.from_numpy((np.zeros(len(self._m.f), np.int64) if pf is None else pf).copy())

    def loop_subdivision(self, iterations):
        m = self._m
        for _ in range(int(iterations)):
            m = m.subdivide()
        return Sphere(_mesh=m)

    def get_vertex_resolution(self):
        """Mean over the vertices of the mean distance to the ring (sphere.cpp:610-628)."""
        he, val = self._m.ring()
        v = self._m.v
        nb = v[self._m.dst[np.where(he >= 0, he, 0)]] - v[:, None, :]
        d = np.sqrt((nb * nb).sum(-1)) * (he >= 0)
        return float((d.sum(1) / val).astype(np.float64).mean())

    def scale_vertices(self, scale):
        """Multiplies vertex i by scale[i] (sphere.cpp:924-932)."""
        s = torch.as_tensor(scale).detach().cpu().float().numpy().reshape(-1, 1)
        m = _Mesh.__new__(_Mesh)
        m.__dict__.update(self._m.__dict__)
        m.v = (self._m.v * s).astype(_F32)
        self._m = m

    def get_face_normals(self):
        """(F, 3) float32 unit normals cross(p2 - p1, p0 - p1) of the walk-order vertices
        (sphere.cpp:466-484)."""
        p = self._m.v[self._face_walk()]
        a, b = p[:, 2] - p[:, 1], p[:, 0] - p[:, 1]
        n = np.stack([a[:, 1] * b[:, 2] - a[:, 2] * b[:, 1], a[:, 2] * b[:, 0] - a[:, 0] * b[:, 2],
                      a[:, 0] * b[:, 1] - a[:, 1] * b[:, 0]], 1).astype(_F32)
        nrm = np.sqrt(n[:, 0] * n[:, 0] + n[:, 1] * n[:, 1] + n[:, 2] * n[:, 2]).astype(_F32)
        return torch.from_numpy((n / nrm[:, None]).astype(_F32))


def generate_icosphere(order=0):
    """Icosphere of the given order as a `Sphere` (package/layers/util/icosphere_functions.py:9-14)."""
    return Sphere.generate_icosphere(order)
