"""Voting resample and cube2rect: oracle against the reference's vectors (CPU), kernels against both (GPU).

Voting resample is integer work: everything is compared exactly.  cube2rect exists only as a CUDA
kernel in the reference; its vectors (tests/golden/cube2rect_ref.npz) were recorded from that kernel
on a GPU.  The library's kernel spells the same arithmetic and must reproduce them bit for bit; the
C oracle uses the host's sin / cos, which moves a sample position by a few ulps of cube_dim, so it
is compared with a tolerance: bilinear 8 * eps * cube_dim * max|cube| (eps of the image's type),
nearest exact except for at most 0.5 % of the pixels (samples that sit on a rounding boundary).
Pixels that look along an edge of the cube (two of |x|, |y|, |z| equal to within 1e-5: whole columns
of them for image widths that are multiples of 8) are left out of the oracle comparisons: which of
the two faces they read hangs on the last bit of sin / cos.
"""
import importlib
import os

import numpy as np
import pytest
import torch

from oracle import oracle

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _vote_cases():
    z = np.load(os.path.join(GOLD, "extras.npz"))
    names = sorted({k.split("/")[1] for k in z.files if k.startswith("vote/")})
    return z, names


def _cube_cases():
    z = np.load(os.path.join(GOLD, "cube2rect_ref.npz"))
    return z, sorted({k.split("/")[0] for k in z.files})


def _off_edge(RH, RW):
    """True for the pixels whose direction is not (nearly) on an edge of the cube."""
    xr, yr = np.arange(RW, dtype=np.float64), np.arange(RH, dtype=np.float64)
    lon = (2 * np.pi * (xr - RW / 2) / RW)[None, :]
    lat = (np.pi * (yr - (RH - 1) / 2) / (RH - 1))[:, None]
    a = np.sort(np.abs(np.stack([np.cos(lat) * np.sin(lon), -np.sin(lat) * np.ones_like(lon),
                                 np.cos(lat) * np.cos(lon)])), axis=0)
    return (a[2] - a[1]) > 1e-5 * a[2]


def _cube_tol(cube):
    return 8 * torch.finfo(cube.dtype).eps * cube.shape[1] * cube.abs().max().item()


def _bindings():
    ops = importlib.import_module("mappedconvolutions_b200.ops")
    from mappedconvolutions_b200 import host
    out = [("ctypes", ops)]
    if host.COMPILED:
        out.append(("compiled", host.impl))
    return out


# ------------------------------------------------------------------------------------------ CPU

def test_voting_oracle_equals_the_reference_vectors():
    z, names = _vote_cases()
    assert len(names) == 5
    for n in names:
        OH, OW, NC = (int(v) for v in z["vote/%s/args" % n])
        got = oracle.voting_resample_to_map(torch.from_numpy(z["vote/%s/labels" % n]),
                                            torch.from_numpy(z["vote/%s/map" % n]), OH, OW, NC)
        assert np.array_equal(got.numpy(), z["vote/%s/out" % n]), n


def test_voting_oracle_known_answer():
    # three pixels vote 2, 2, 1 for target (0, 0); one votes 3 for (1, 0); (0, 1) and (1, 1) get nothing
    labels = torch.tensor([[[[2, 2, 1, 3]]]])
    smap = torch.tensor([[[0, 0], [0, 0], [0, 0], [1, 0]]]).view(1, 4, 2)
    out = oracle.voting_resample_to_map(labels, smap, 2, 2, 4)
    assert out.tolist() == [[[[2, 3], [0, 0]]]]
    # a tie goes to the smaller label
    labels = torch.tensor([[[[3, 1, 1, 3]]]])
    smap = torch.zeros(1, 4, 2, dtype=torch.int64)
    assert oracle.voting_resample_to_map(labels, smap, 1, 1, 4).item() == 1


def _check_cube_oracle(z, n):
    cube = torch.from_numpy(z[n + "/cube"])
    RH, RW = (int(v) for v in z[n + "/shape"])
    keep = _off_edge(RH, RW)
    assert keep.mean() > 0.85
    bil = oracle.cube2rect(cube, RH, RW, 1).numpy()
    ref = z[n + "/bilinear"]
    assert np.abs(bil - ref)[:, keep].max() <= _cube_tol(cube), n
    near = oracle.cube2rect(cube, RH, RW, 0).numpy()
    ref = z[n + "/nearest"]
    assert (near != ref)[:, keep].mean() <= 0.005, n


def test_cube2rect_oracle_matches_the_reference_kernel_vectors():
    z, names = _cube_cases()
    assert len(names) == 5
    for n in names:
        _check_cube_oracle(z, n)


def test_cube2rect_oracle_constant_faces():
    # each face filled with its own index: nearest sampling returns the face every direction hits
    D = 4
    cube = torch.arange(6, dtype=torch.float32).repeat_interleave(D).expand(1, D, 6 * D).contiguous()
    rect = oracle.cube2rect(cube, 9, 16, 0)[0]
    assert rect[0].eq(4).all() and rect[-1].eq(5).all()          # poles: +y on top, -y at the bottom
    mid = rect[4]
    assert mid[8] == 2 and mid[0] == 0 and mid[4] == 1 and mid[12] == 3   # lon 0 -> +z, -pi -> -z, -+pi/2 -> -+x
    # bilinear sampling of constant faces stays within the faces' value range
    rb = oracle.cube2rect(cube, 9, 16, 1)
    assert rb.min() >= -1e-5 and rb.max() <= 5 + 1e-5


def test_grid_convolution_layers_equal_the_references():
    """Seeded construction gives the reference's parameters bit for bit; outputs and gradients agree
    with the reference's im2col + GEMM code to 1e-5 of the largest magnitude (float32, another
    summation order)."""
    from mappedconvolutions_b200 import nn as mnn
    cases = importlib.import_module("golden.make_golden_extras").GRID_CASES
    z = np.load(os.path.join(GOLD, "extras.npz"))
    for name, (cls, kw, shape) in cases.items():
        torch.manual_seed(0)
        layer = getattr(mnn, cls)(**kw)
        assert np.array_equal(layer.weight.detach().numpy(), z["grid/%s/weight" % name]), name
        assert np.array_equal(layer.bias.detach().numpy(), z["grid/%s/bias" % name]), name
        x = torch.from_numpy(z["grid/%s/x" % name]).requires_grad_(True)
        y = layer(x)
        assert tuple(y.shape) == z["grid/%s/y" % name].shape, name
        y.backward(torch.from_numpy(z["grid/%s/gy" % name]))
        for got, key in ((y, "y"), (x.grad, "gx"), (layer.weight.grad, "gw"), (layer.bias.grad, "gb")):
            want = z["grid/%s/%s" % (name, key)]
            assert np.abs(got.detach().numpy() - want).max() <= 1e-5 * max(1.0, np.abs(want).max()), (name, key)


# ------------------------------------------------------------------------------------------ GPU

@pytest.mark.gpu
def test_voting_kernel_equals_the_reference_vectors():
    z, names = _vote_cases()
    for bname, ops in _bindings():
        for n in names:
            OH, OW, NC = (int(v) for v in z["vote/%s/args" % n])
            got = ops.voting_resample_to_map(torch.from_numpy(z["vote/%s/labels" % n]).cuda(),
                                             torch.from_numpy(z["vote/%s/map" % n]).cuda(), OH, OW, NC)
            assert got.dtype == torch.int64
            assert np.array_equal(got.cpu().numpy(), z["vote/%s/out" % n]), (bname, n)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(1, 1, 512, 1024, 128, 256, 21), (4, 1, 256, 512, 300, 300, 40),
                                   (2, 2, 100, 77, 50, 60, 3), (1, 1, 1, 1, 1, 1, 1)])
def test_voting_kernel_equals_the_oracle(shape):
    B, C, IH, IW, OH, OW, NC = shape
    g = torch.Generator().manual_seed(sum(shape))
    labels = torch.randint(0, NC, (B, C, IH, IW), generator=g)
    labels[0, 0, 0, 0] = NC + 3 if NC > 1 else 0          # a label outside the candidates is ignored
    smap = torch.stack([torch.randint(-2, OW + 2, (IH, IW), generator=g),
                        torch.randint(-2, OH + 2, (IH, IW), generator=g)], -1).contiguous()
    want = oracle.voting_resample_to_map(labels, smap, OH, OW, NC)
    for bname, ops in _bindings():
        got = ops.voting_resample_to_map(labels.cuda(), smap.cuda(), OH, OW, NC)
        assert torch.equal(got.cpu(), want), bname


@pytest.mark.gpu
def test_voting_argument_checks():
    for bname, ops in _bindings():
        lab = torch.zeros(1, 1, 4, 4, dtype=torch.int64, device="cuda")
        with pytest.raises(RuntimeError):
            ops.voting_resample_to_map(lab.float(), torch.zeros(4, 4, 2, dtype=torch.int64, device="cuda"), 2, 2, 3)
        with pytest.raises(RuntimeError):
            ops.voting_resample_to_map(lab, torch.zeros(4, 5, 2, dtype=torch.int64, device="cuda"), 2, 2, 3)
        with pytest.raises(RuntimeError):
            ops.voting_resample_to_map(lab, torch.zeros(4, 4, 2, dtype=torch.int64, device="cuda"), 2, 2, 0)


@pytest.mark.gpu
def test_cube2rect_kernel_reproduces_the_reference_kernel_bit_for_bit():
    z, names = _cube_cases()
    for bname, ops in _bindings():
        for n in names:
            cube = torch.from_numpy(z[n + "/cube"]).cuda()
            RH, RW = (int(v) for v in z[n + "/shape"])
            for interp, tag in ((0, "nearest"), (1, "bilinear")):
                got = ops.cube2rect(cube, RH, RW, interp).cpu().numpy()
                assert got.dtype == z[n + "/" + tag].dtype
                assert np.array_equal(got, z[n + "/" + tag]), (bname, n, tag, np.abs(got - z[n + "/" + tag]).max())


@pytest.mark.gpu
@pytest.mark.parametrize("case", [(3, 64, 256, 512, torch.float32), (1, 7, 31, 50, torch.float64),
                                  (2, 256, 512, 1024, torch.float32)])
def test_cube2rect_kernel_against_the_oracle(case):
    C, D, RH, RW, dt = case
    g = torch.Generator().manual_seed(C * D + RH)
    cube = torch.randn(C, D, 6 * D, generator=g, dtype=dt)
    keep = torch.from_numpy(_off_edge(RH, RW))
    for bname, ops in _bindings():
        bil = ops.cube2rect(cube.cuda(), RH, RW, 1).cpu()
        want = oracle.cube2rect(cube, RH, RW, 1)
        assert (bil - want).abs()[:, keep].max() <= _cube_tol(cube), bname
        near = ops.cube2rect(cube.cuda(), RH, RW, 0).cpu()
        assert (near != oracle.cube2rect(cube, RH, RW, 0))[:, keep].float().mean() <= 0.005, bname


@pytest.mark.gpu
def test_cube_to_rect_of_the_util_package_and_argument_checks():
    from mappedconvolutions_b200.util import spherical_projections as sp
    cube = torch.randn(2, 8, 48, device="cuda")
    ops = importlib.import_module("mappedconvolutions_b200.ops")
    assert torch.equal(sp.cube_to_rect(cube, 16, 32, "bilinear"), ops.cube2rect(cube, 16, 32, 1))
    assert torch.equal(sp.cube_to_rect(cube, 16, 32), ops.cube2rect(cube, 16, 32, 0))
    for bname, o in _bindings():
        with pytest.raises(RuntimeError):
            o.cube2rect(cube[:, :, :40], 16, 32, 0)
        with pytest.raises(RuntimeError):
            o.cube2rect(cube.half(), 16, 32, 0)
        with pytest.raises(RuntimeError):
            o.cube2rect(cube, 16, 32, 2)
