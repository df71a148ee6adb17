"""The utility surface (mesh, map builders, conversions, grids) against vectors produced by the
reference's own code (tests/golden/util.npz, written by tests/golden/make_golden_util.py).  Large
results are compared through SHA-256 digests of their bytes, so equality there means bit for bit."""
import hashlib

import numpy as np
import pytest
import torch

import helpers as H

G = dict(np.load(H.GOLDEN + "/util.npz"))


def digest(t):
    a = np.ascontiguousarray(t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else t)
    return np.frombuffer(hashlib.sha256(a.tobytes()).digest(), dtype=np.uint8)


def same(got, key):
    want = G[key]
    got = got.detach().cpu().contiguous() if isinstance(got, torch.Tensor) else got
    if key.endswith("_sha") or (want.dtype == np.uint8 and want.shape == (32,)):
        assert np.array_equal(digest(got), want), key
    else:
        g = got.numpy() if isinstance(got, torch.Tensor) else np.asarray(got)
        assert g.shape == want.shape, (key, g.shape, want.shape)
        assert g.dtype == want.dtype, (key, g.dtype, want.dtype)
        assert np.array_equal(g, want, equal_nan=True), (key, np.abs(g.astype(np.float64) - want).max())


@pytest.mark.parametrize("order", range(8))
def test_icosphere_is_the_reference_mesh(order):
    """Vertices (float32, bit for bit), faces, the three adjacency tables, barycentres and normals
    of generate_icosphere(order) for orders 0-7 (sphere.cpp:512-539, :811-912, :631-680)."""
    from mappedconvolutions_b200.util import generate_icosphere
    s = generate_icosphere(order)
    assert s.num_vertices() == 10 * 4 ** order + 2 and s.num_faces() == 20 * 4 ** order
    p = "sphere%d/" % order
    same(s.get_vertices(), p + "vertices")
    same(s.get_all_face_vertex_indices(), p + "faces")
    same(s.get_adjacent_vertex_indices_to_vertices(), p + "adj_vv")
    same(s.get_adjacent_face_indices_to_vertices(), p + "adj_fv")
    same(s.get_adjacent_face_indices_to_faces(), p + "adj_ff")
    same(s.get_face_barycenters(), p + "barycenters")
    same(s.get_face_normals(), p + "normals")
    if order >= 1:
        same(s.get_original_face_indices(), p + "original_faces")
    # the reference sums this in an OpenMP reduction (order not fixed): tolerance
    assert abs(s.get_vertex_resolution() - float(G[p + "resolution"])) <= 1e-6


def test_projection_maps_equal_the_references():
    """get_projection_map for the three projections incl. stride and dilation, the perspective and
    cube-map kernels (spherical_projections.py:12-35, :38-196, :258-307); the 512 x 1024 gnomonic
    map of the headline benchmark through its digest."""
    from mappedconvolutions_b200 import util as U
    same(U.get_projection_map((16, 32), (3, 3), "gnomonic"), "proj/gnomonic_16x32_3x3")
    same(U.get_projection_map((16, 32), (5, 3), "gnomonic", 2), "proj/gnomonic_16x32_5x3_s2")
    same(U.get_projection_map((16, 32), (3, 3), "equirectangular"), "proj/equirect_16x32_3x3")
    same(U.get_projection_map((16, 32), (3, 5), "grid", 1, 2), "proj/grid_16x32_3x5_d2")
    same(U.get_projection_map((512, 1024), (3, 3), "gnomonic"), "proj/gnomonic_512x1024_3x3_sha")
    same(U.get_perspective_projection_map((6, 7), (3, 3), 1, 2), "proj/perspective_6x7_3x3_d2")
    same(U.get_reverse_cube_projection_map(4, (3, 3)), "proj/cube4_3x3")
    same(U.reverse_cubemap_projection_map(4, (3, 3)), "proj/reverse_cubemap4_3x3")
    same(U.perspective_resampling(60.0, 8, 6, 30.0), "proj/perspective_resampling")


def test_conversions_and_grids_equal_the_references():
    from mappedconvolutions_b200 import util as U
    xyz = torch.from_numpy(G["conv/xyz"])
    lonlat = U.convert_3d_to_spherical(xyz)
    same(lonlat, "conv/lonlat")
    same(U.convert_spherical_to_image(lonlat, (32, 64)), "conv/image")
    same(U.convert_spherical_to_3d(lonlat), "conv/back3d")
    uv, idx = U.convert_3d_to_cube(xyz, 8)
    same(uv, "conv/cube_uv")
    same(idx, "conv/cube_idx")
    same(U.convert_cube_to_3d(uv, idx[..., 0], 8), "conv/cube_to_3d")
    same(U.convert_cubemap_tuple_to_image(uv, idx, 8), "conv/cubemap_image")
    uv2, idx2 = U.convert_spherical_to_cube(lonlat[:64], 8)   # (the last rows are exact ties)
    assert torch.equal(idx2, idx[:64]) and (uv2 - uv[:64]).abs().max().item() <= 1e-4
    lat, lon, rla, rlo = U.equirectangular_meshgrid((8, 16))   # the grids.py one: latitude ascending
    same(lat, "grid/lat")
    same(lon, "grid/lon")
    assert np.array_equal(np.array([rla, rlo]), G["grid/res"])
    assert U.get_equirectangular_grid_resolution((8, 16)) == (rla, rlo)
    v, u, index = U.cube_meshgrid(4)
    same(v, "grid/cube_v")
    same(u, "grid/cube_u")
    same(index, "grid/cube_index")
    y, x = U.cartesian_meshgrid((3, 4))
    assert torch.equal(x[0], torch.arange(4.)) and torch.equal(y[:, 0], torch.arange(3.))


def test_icosphere_maps_equal_the_references():
    """image_to_sphere_resample_map with the reference's signature (image_shape, icosphere, source),
    gnomonic kernels at the vertices, the face pooling map (icosphere_functions.py:20-25, :135-223,
    :383-405; mesh_functions.py:22-31)."""
    from mappedconvolutions_b200 import util as U
    s2, s3 = U.generate_icosphere(2), U.generate_icosphere(3)
    assert np.array_equal(np.array([U.compute_num_vertices(o) for o in range(8)]), G["ico/num_vertices"])
    same(U.image_to_sphere_resample_map((64, 128), s3, "vertex"), "ico/image_to_sphere_vertex")
    same(U.image_to_sphere_resample_map((64, 128), s3, "face"), "ico/image_to_sphere_face")
    same(U.image_to_sphere_resample_map((512, 1024), U.generate_icosphere(7)),
         "ico/image_to_sphere_512x1024_l7_sha")
    res = s2.get_vertex_resolution()
    got = U.gnomonic_kernel_from_sphere(s2, 3, 3, res, res, "vertex")
    want = torch.from_numpy(G["ico/gnomonic_kernel_s2"])
    assert got.shape == want.shape and (got - want).abs().max().item() <= 2e-6  # res differs by 1e-8
    same(U.get_downsample_map(s3, 2), "ico/downsample_map_3_2")
    assert torch.equal(U.vertices_to_equirectangular_resample_map(s3, (64, 128)).view(1, -1, 2),
                       U.image_to_sphere_resample_map((64, 128), s3))


def test_tensor_helpers_equal_the_references():
    from mappedconvolutions_b200 import util as U
    x, i2, i1 = (torch.from_numpy(G["util/" + k]) for k in ("x", "i2", "i1"))
    same(U.batched_index_select(x, 2, i2), "util/select2")
    same(U.batched_index_select(x, -1, i1), "util/select1")
    same(U.batched_scatter(x, 2, i1), "util/scatter")


def test_benchmark_one_ring_maps_come_from_the_reference_mesh():
    """The 7-tap kernel and pooling maps of the icosphere configurations: tap 0 the vertex, taps 1-6
    the ring of get_adjacent_vertex_indices_to_vertices, 12 rows with a repeated first neighbour."""
    from mappedconvolutions_b200 import util as U
    ring = torch.from_numpy(G["sphere2/adj_vv"])
    km = U.vertex_kernel_map(2)
    assert km.shape == (1, 162, 7, 2) and km.dtype == torch.float32
    assert torch.equal(km[0, :, 0, 0], torch.arange(162.)) and torch.equal(km[0, :, 1:, 0], ring.float())
    assert (km[..., 1] == 0).all()
    assert int((km[0, :, 6, 0] == km[0, :, 1, 0]).sum()) == 12
    pm = U.pooling_map(2)
    assert pm.shape == (1, 42, 7, 2) and torch.equal(pm[0], km[0, :42])


def test_reference_surface_names_are_exported():
    """Every public function of the reference's util modules this library carries, under both
    package names."""
    import mapped_convolution.util as A
    import mapped_convolutions.util as B
    names = """generate_icosphere compute_num_vertices resample_vertex_to_rect resample_rgb_to_vertex
        resample_cube_to_vertex gnomonic_kernel gnomonic_kernel_from_sphere vertex_to_vertex_kernel_map
        faces_to_equirectangular_resample_map vertices_to_equirectangular_resample_map
        sphere_to_image_resample_map sphere_to_cube_resample_map sphere_to_samples_resample_map
        image_to_sphere_resample_map get_downsample_map vertices_to_faces faces_to_vertices knn
        get_projection_map get_reverse_cube_projection_map get_perspective_projection_map
        grid_projection_map perspective_projection_map equirectangular_meshgrid
        reverse_equirectangular_projection_map reverse_gnomonic_projection_map cube_to_rect cube_to_3d
        reverse_cubemap_projection_map cubemap_idx_to_xy perspective_resampling time_cuda
        batched_index_select batched_scatter convert_spherical_to_image convert_3d_to_spherical
        convert_spherical_to_3d convert_3d_to_cube convert_spherical_to_cube convert_cube_to_3d
        convert_cubemap_tuple_to_image get_equirectangular_grid_resolution cube_meshgrid_resolution
        cube_meshgrid cartesian_meshgrid""".split()
    for n in names:
        assert callable(getattr(A, n)) and getattr(B, n) is getattr(A, n), n


@pytest.mark.gpu
def test_point_location_on_the_gpu_matches_the_reference_search():
    """mc_sphere_locate (the device-side form of Sphere::getPlanarConvolutionOperatorFromSamples,
    sphere.cpp:1116-1270) through the map builders that use it.  Vertex triples must equal the
    reference's wherever the sample is not within 2e-3 of a face border (there the first face in
    search order that passes the -1e-3 test wins, which last-bit differences of sin / cos can tip);
    weights within 1e-5; in every case the weights reproduce the sample from the vertices."""
    from mappedconvolutions_b200 import util as U

    def check(V, W, kv, kw, min_same):
        wv, ww = torch.from_numpy(G[kv]), torch.from_numpy(G[kw])
        V, W = V.cpu(), W.cpu()
        assert V.shape == wv.shape and W.shape == ww.shape and V.dtype == wv.dtype
        agree = (V == wv).all(-1).all(-1)
        interior = ww.min(-1).values > 2e-3
        assert agree[interior].all(), "vertex triple differs inside a face"
        assert agree.float().mean().item() >= min_same
        assert (W - ww)[agree].abs().max().item() <= 1e-5
        assert (W.sum(-1) - 1).abs().max().item() <= 1e-5

    V, W = U.sphere_to_image_resample_map(3, (24, 48))
    check(V, W, "locate/image_24x48_o3_V", "locate/image_24x48_o3_W", 0.98)
    Vn, Wn = U.sphere_to_image_resample_map(3, (24, 48), True)
    wn = torch.from_numpy(G["locate/image_24x48_o3_nearest_W"])
    assert ((Wn.cpu() == wn).all(-1).float().mean().item()) >= 0.98
    assert torch.equal(Wn.sum(-1).cpu(), torch.ones(24, 48))
    s2 = U.generate_icosphere(2)
    V, W = U.vertex_to_vertex_kernel_map(s2, 3, 3, 3)
    assert V.shape == (1, 162, 9, 3, 2)
    check(V, W, "locate/v2v_s2_o3_V", "locate/v2v_s2_o3_W", 0.97)
    V, W = U.sphere_to_cube_resample_map(2, 6)
    check(V, W, "locate/cube6_o2_V", "locate/cube6_o2_W", 0.98)
    V, W = U.sphere_to_image_resample_map(5, (64, 128))
    ww = torch.from_numpy(G["locate/image_64x128_o5_W"])
    assert ((W.cpu() - ww).abs().max(-1).values <= 1e-5).float().mean().item() >= 0.98
    # the weights interpolate the vertex positions back to the sample direction
    verts = U.generate_icosphere(5).get_vertices()
    lat, lon, _, _ = U.equirectangular_meshgrid((64, 128))
    want = U.convert_spherical_to_3d(torch.stack((lon, lat), -1))
    got = (verts[V[..., 0].long().cpu()] * W.cpu().unsqueeze(-1)).sum(-2)
    got = got / got.norm(dim=-1, keepdim=True)
    assert (got - want).abs().max().item() <= 2e-3
