"""CPU: the plain-C oracle against the golden vectors produced by the reference's own CPU code
(tests/golden/make_golden.py).  This is what pins the oracle."""
import pytest
import torch

import helpers as H
from oracle import oracle

KAT = H.load_cases("kat.npz")
RND = H.load_cases("random_small.npz")
IMPL = H.Impl(oracle)


def _kat_forward(ops, c, dev="cpu"):
    """Replays one recorded known-answer test through an op module; returns output and grads."""
    t = lambda v: None if v is None else v.to(dev)
    x, m, iw = t(c["input"]), t(c["sample_map"]), t(c.get("interp_weights"))
    interp, layer = c["interp"], c["layer"]
    ones = torch.ones_like(t(c["output"]))
    if layer == "MappedConvolution":
        w, b, K = t(c["weight"]), t(c["bias"]), c["kernel_size"]
        if iw is None:
            y = ops.mapped_conv_forward(x, m, w, b, K, interp)
            g = ops.mapped_conv_backward(ones, m, x, w, b, K, interp)
        else:
            y = ops.weighted_mapped_conv_forward(x, m, iw, w, b, K, interp)
            g = ops.weighted_mapped_conv_backward(ones, m, iw, x, w, b, K, interp)
        return dict(output=y, grad_input=g[0], grad_weight=g[1], grad_bias=g[2])
    if layer == "MappedTransposedConvolution":
        w, b, K = t(c["weight"]), t(c["bias"]), c["kernel_size"]
        y = ops.mapped_transposed_conv_forward(x, m, w, b, c["oh"], c["ow"], K, interp)
        g = ops.mapped_transposed_conv_backward(ones, m, x, w, b, K, interp)
        return dict(output=y, grad_input=g[0], grad_weight=g[1], grad_bias=g[2])
    if layer == "MappedMaxPool":
        y, idx = ops.mapped_max_pool(x, m, c["kernel_size"], interp)
        gx = ops.mapped_max_unpool(ones, idx, m, x.shape[2], x.shape[3], c["kernel_size"], interp)
        return dict(output=y, grad_input=gx)
    if layer == "MappedAvgPool":
        y = ops.mapped_avg_pool(x, m, c["kernel_size"], interp)
        gx = ops.mapped_avg_unpool(ones, m, x.shape[2], x.shape[3], c["kernel_size"], interp)
        return dict(output=y, grad_input=gx)
    if layer == "Unresample":
        if iw is None:
            y = ops.resample_from_map(x, m, interp)
            gx = ops.resample_to_map(ones, m, x.shape[2], x.shape[3], interp)
        else:
            y = ops.weighted_resample_from_map(x, m, iw, interp)
            gx = ops.weighted_resample_to_map(ones, m, iw, x.shape[2], x.shape[3], interp)
        return dict(output=y, grad_input=gx)
    raise AssertionError(layer)


def check_kat(ops, c, name, dev="cpu", tol=1e-12):
    got = _kat_forward(ops, c, dev)
    # the literal tensor the reference's test asserts against, with that test's own tolerance
    assert torch.allclose(got["output"].cpu(), c["expected"], rtol=1e-5, atol=1e-8), name
    for k, v in got.items():
        H.assert_close(v, c[k], tol, "%s/%s" % (name, k))


@pytest.mark.parametrize("name", sorted(KAT))
def test_oracle_reproduces_reference_kat(name):
    check_kat(oracle, KAT[name], name)


def test_kat_count():
    # 6 conv + 3 transposed conv + 5 pooling + 10 resample CPU tests of the reference
    assert len(KAT) == 24


@pytest.mark.parametrize("name", sorted(n for n in RND if n.startswith("conv_")))
def test_oracle_conv_random(name):
    c = RND[name]
    H.compare_case(H.run_conv(IMPL, c), c, H.TOL[c["input"].dtype] , name)


@pytest.mark.parametrize("name", sorted(n for n in RND if n.startswith("tconv_")))
def test_oracle_tconv_random(name):
    c = RND[name]
    H.compare_case(H.run_conv(IMPL, c, transposed=True), c, H.TOL[c["input"].dtype], name)


@pytest.mark.parametrize("name", sorted(n for n in RND if n.startswith("pool_f")))
def test_oracle_pool_random(name):
    c = RND[name]
    H.compare_case(H.run_pool(IMPL, c), c, H.TOL[c["input"].dtype], name)


@pytest.mark.parametrize("name", sorted(n for n in RND if n.startswith("resample_")))
def test_oracle_resample_random(name):
    c = RND[name]
    H.compare_case(H.run_resample(IMPL, c), c, H.TOL[c["input"].dtype], name)


def test_oracle_max_pool_cpu_start_value():
    """With the reference CPU build's start value the oracle reproduces its output everywhere,
    including the windows it reports as index -1; with the CUDA build's start value (-FLT_MAX)
    it agrees wherever the CPU build found a tap."""
    c = RND["pool_cpu_init_f32"]
    y, idx = oracle.mapped_max_pool(c["input"], c["sample_map"], c["K"], c["interp"], cuda_init=False)
    assert torch.equal(y, c["max_output"]) and torch.equal(idx, c["max_idx"])
    assert (c["max_idx"] < 0).any()
    y2, idx2 = oracle.mapped_max_pool(c["input"], c["sample_map"], c["K"], c["interp"], cuda_init=True)
    ok = c["max_idx"] >= 0
    assert torch.equal(y2[ok], c["max_output"][ok]) and torch.equal(idx2[ok], c["max_idx"][ok])
    assert (idx2 >= 0).all()


def test_oracle_config1():
    c = H.load_cases("config1.npz")["config1"]
    H.compare_case(H.run_conv(IMPL, c), c, 1e-5, "config1")


@pytest.mark.parametrize("D,M,N,k", [(3, 2000, 500, 9), (2, 800, 800, 4), (5, 300, 64, 16)])
def test_oracle_knn_against_independent_searches(D, M, N, k):
    """The reference ships no CPU k-NN and no k-NN test, so its semantics are cross-checked against
    two independent exact searches instead: SciPy's k-d tree and a float64 brute force.  Same
    neighbour sets, 1-based indices, ascending Euclidean distances (1e-5 relative: the oracle
    accumulates in float32 like the reference's kernel)."""
    import numpy as np
    from scipy.spatial import cKDTree
    g = torch.Generator().manual_seed(D * 1000 + k)
    ref = torch.randn(1, D, M, generator=g)
    q = torch.randn(1, D, N, generator=g)
    idx, dist = oracle.knn_forward(ref, q, k)
    idx, dist = idx[0].numpy(), dist[0].numpy()                     # (k, N)
    assert idx.min() >= 1 and idx.max() <= M
    assert (np.diff(dist, axis=0) >= 0).all()
    r64, q64 = ref[0].double().numpy().T, q[0].double().numpy().T   # (M, D), (N, D)
    tree_d, tree_i = cKDTree(r64).query(q64, k=k)
    brute = np.sqrt(((q64[:, None, :] - r64[None, :, :]) ** 2).sum(-1))
    brute_i = np.argsort(brute, axis=1, kind="stable")[:, :k]
    for n in range(N):
        assert set(idx[:, n] - 1) == set(tree_i[n]) == set(brute_i[n]), n
    np.testing.assert_allclose(dist.T, tree_d, rtol=1e-5, atol=1e-6)


# ---- k-NN against the reference's own CUDA kernels -----------------------------------------------
# tests/golden/knn_ref.npz holds outputs of the reference's knn_forward built from its sources for
# sm_100a and run on a B200 (tests/golden/make_golden_knn.py).  The reference is in bounds only for
# M == k, so every case has M == k: the whole reference set is returned, sorted - which pins the
# distance arithmetic (the fma chain over dimensions), the ordering and tie-break by index, the
# 1-based numbering and the square root.
KNN_REF = H.load_cases("knn_ref.npz")


@pytest.mark.parametrize("name", sorted(KNN_REF))
def test_oracle_knn_equals_the_reference_kernels(name):
    c = KNN_REF[name]
    idx, dist = oracle.knn_forward(c["ref"], c["query"], int(c["k"]))
    assert torch.equal(idx, c["idx"]), "%s: indices differ at %d places" % (name, (idx != c["idx"]).sum())
    assert torch.equal(dist, c["dist"]), "%s: distances not bit-identical" % name
    assert idx.min().item() == 1 and idx.max().item() == int(c["k"])
