"""Generate tests/golden/util.npz by running the REFERENCE's own utility code: the pure-torch map
builders of package/layers/util (loaded as loose modules) and its Sphere class
(oracle/_ref/_mapped_convolution_ext/_sphere.so, built by oracle/build_ref.py).

    MC_REFERENCE_ROOT=<reference checkout> python tests/golden/make_golden_util.py

Run by hand when the fixtures need refreshing; the tests only read the .npz file, never the
reference.  Large results (the level 5-7 meshes, the 512 x 1024 gnomonic map) are stored as
SHA-256 digests of their raw bytes.
"""
import hashlib
import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.dont_write_bytecode = True

from oracle import ref  # noqa: E402


def digest(t):
    a = np.ascontiguousarray(t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else t)
    return np.frombuffer(hashlib.sha256(a.tobytes()).digest(), dtype=np.uint8).copy()


def load_reference_util(ref_root):
    """The reference's util modules as a synthetic package `refutil`, with the compiled modules they
    import replaced: _sphere by the reference's own build, the CUDA-only ones by empty stand-ins,
    the layer classes (not called here) by placeholders."""
    ext = types.ModuleType("_mapped_convolution_ext")
    ext._sphere = ref.load("_sphere")
    ext._cube2rect = types.ModuleType("_mapped_convolution_ext._cube2rect")
    ext._knn = types.ModuleType("_mapped_convolution_ext._knn")
    sys.modules.update({"_mapped_convolution_ext": ext, "_mapped_convolution_ext._sphere": ext._sphere,
                        "_mapped_convolution_ext._cube2rect": ext._cube2rect,
                        "_mapped_convolution_ext._knn": ext._knn})
    mc = types.ModuleType("mapped_convolution")
    mc.nn = types.ModuleType("mapped_convolution.nn")
    mc.nn.Resample = mc.nn.Unresample = object
    sys.modules.update({"mapped_convolution": mc, "mapped_convolution.nn": mc.nn})
    pkg = types.ModuleType("refutil")
    pkg.__path__ = [os.path.join(ref_root, "package", "layers", "util")]
    sys.modules["refutil"] = pkg
    names = ("conversions", "grids", "spherical_projections", "icosphere_functions", "mesh_functions", "util")
    return types.SimpleNamespace(**{n: importlib.import_module("refutil." + n) for n in names})


def main():
    ref_root = os.environ.get("MC_REFERENCE_ROOT")
    assert ref_root and os.path.isdir(ref_root), "set MC_REFERENCE_ROOT to the reference checkout"
    R = load_reference_util(ref_root)
    S = ref.load("_sphere").Sphere
    out = {}
    # ---- mesh ------------------------------------------------------------------------------------
    for order in range(0, 8):
        s = S.generate_icosphere(order)
        fields = dict(vertices=s.get_vertices(), faces=s.get_all_face_vertex_indices(),
                      adj_vv=s.get_adjacent_vertex_indices_to_vertices(),
                      adj_fv=s.get_adjacent_face_indices_to_vertices(),
                      adj_ff=s.get_adjacent_face_indices_to_faces(),
                      barycenters=s.get_face_barycenters(), normals=s.get_face_normals())
        if order >= 1:
            fields["original_faces"] = s.get_original_face_indices()
        for k, v in fields.items():
            out["sphere%d/%s" % (order, k)] = v.numpy() if order <= 2 else digest(v)
        out["sphere%d/resolution" % order] = np.float64(s.get_vertex_resolution())
    # ---- projection maps -------------------------------------------------------------------------
    sp = R.spherical_projections
    for name, args in (("gnomonic_16x32_3x3", ((16, 32), (3, 3), "gnomonic")),
                       ("gnomonic_16x32_5x3_s2", ((16, 32), (5, 3), "gnomonic", 2)),
                       ("equirect_16x32_3x3", ((16, 32), (3, 3), "equirectangular")),
                       ("grid_16x32_3x5_d2", ((16, 32), (3, 5), "grid", 1, 2))):
        out["proj/" + name] = sp.get_projection_map(*args).contiguous().numpy()
    out["proj/gnomonic_512x1024_3x3_sha"] = digest(sp.get_projection_map((512, 1024), (3, 3), "gnomonic").contiguous())
    out["proj/perspective_6x7_3x3_d2"] = sp.get_perspective_projection_map((6, 7), (3, 3), 1, 2).contiguous().numpy()
    out["proj/cube4_3x3"] = sp.get_reverse_cube_projection_map(4, (3, 3)).contiguous().numpy()
    out["proj/reverse_cubemap4_3x3"] = sp.reverse_cubemap_projection_map(4, (3, 3)).contiguous().numpy()
    out["proj/perspective_resampling"] = sp.perspective_resampling(60.0, 8, 6, 30.0).numpy()
    g = torch.Generator().manual_seed(0)
    # ---- conversions and grids -------------------------------------------------------------------
    cv = R.conversions
    xyz = torch.randn(64, 3, generator=g)
    xyz = torch.cat([xyz, torch.tensor([[1., 1., 0.5], [-1., 1., 1.], [0.5, -1., -1.]])], 0)
    lonlat = cv.convert_3d_to_spherical(xyz)
    uv, idx = cv.convert_3d_to_cube(xyz, 8)
    out.update({"conv/xyz": xyz.numpy(), "conv/lonlat": lonlat.numpy(),
                "conv/image": cv.convert_spherical_to_image(lonlat, (32, 64)).numpy(),
                "conv/back3d": cv.convert_spherical_to_3d(lonlat).numpy(),
                "conv/cube_uv": uv.numpy(), "conv/cube_idx": idx.numpy(),
                "conv/cube_to_3d": cv.convert_cube_to_3d(uv, idx[..., 0], 8).numpy(),
                "conv/cubemap_image": cv.convert_cubemap_tuple_to_image(uv, idx, 8).numpy()})
    lat, lon, rla, rlo = R.grids.equirectangular_meshgrid((8, 16))
    v, u, index = R.grids.cube_meshgrid(4)
    out.update({"grid/lat": lat.contiguous().numpy(), "grid/lon": lon.contiguous().numpy(),
                "grid/res": np.array([rla, rlo]), "grid/cube_v": v.contiguous().numpy(),
                "grid/cube_u": u.contiguous().numpy(), "grid/cube_index": index.contiguous().numpy()})
    # ---- icosphere functions ---------------------------------------------------------------------
    ic = R.icosphere_functions
    s3, s2 = S.generate_icosphere(3), S.generate_icosphere(2)
    out["ico/num_vertices"] = np.array([ic.compute_num_vertices(o) for o in range(8)])
    out["ico/image_to_sphere_vertex"] = ic.image_to_sphere_resample_map((64, 128), s3, "vertex").numpy()
    out["ico/image_to_sphere_face"] = ic.image_to_sphere_resample_map((64, 128), s3, "face").numpy()
    out["ico/image_to_sphere_512x1024_l7_sha"] = digest(
        ic.image_to_sphere_resample_map((512, 1024), S.generate_icosphere(7), "vertex").contiguous())
    res = s2.get_vertex_resolution()
    out["ico/gnomonic_kernel_s2"] = ic.gnomonic_kernel_from_sphere(s2, 3, 3, res, res, "vertex").numpy()
    out["ico/downsample_map_3_2"] = R.mesh_functions.get_downsample_map(s3, 2).numpy()
    # barycentric point location (the reference's host search)
    for nearest in (False, True):
        tag = "_nearest" if nearest else ""
        V, W = ic.sphere_to_image_resample_map(3, (24, 48), nearest)
        out["locate/image_24x48_o3%s_V" % tag] = V.numpy()
        out["locate/image_24x48_o3%s_W" % tag] = W.numpy()
    V, W = ic.vertex_to_vertex_kernel_map(s2, 3, 3, 3, False)
    out["locate/v2v_s2_o3_V"], out["locate/v2v_s2_o3_W"] = V.numpy(), W.numpy()
    V, W = ic.sphere_to_cube_resample_map(2, 6, False)
    out["locate/cube6_o2_V"], out["locate/cube6_o2_W"] = V.numpy(), W.numpy()
    V, W = ic.sphere_to_image_resample_map(5, (64, 128), False)
    out["locate/image_64x128_o5_V_sha"], out["locate/image_64x128_o5_W"] = digest(V), W.numpy()
    # ---- tensor helpers ---------------------------------------------------------------------------
    x = torch.randn(3, 4, 6, generator=g)
    i2 = torch.randint(0, 6, (3, 5), generator=g)
    i1 = torch.randperm(6, generator=g)
    out.update({"util/x": x.numpy(), "util/i2": i2.numpy(), "util/i1": i1.numpy(),
                "util/select2": R.util.batched_index_select(x, 2, i2).numpy(),
                "util/select1": R.util.batched_index_select(x, -1, i1).numpy(),
                "util/scatter": R.util.batched_scatter(x, 2, i1).numpy()})
    np.savez_compressed(os.path.join(HERE, "util.npz"), **out)
    print("wrote util.npz with %d arrays" % len(out))


if __name__ == "__main__":
    main()
