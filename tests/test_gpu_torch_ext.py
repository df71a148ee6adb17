"""The compiled PyTorch C++ extension (csrc_torch/mc_torch_ext.cpp: the reference's pybind surface
on top of the C ABI) against its ctypes twin ops.py: same kernels, so outputs are identical bit for
bit wherever no atomics are involved, and within the float tolerances elsewhere."""
import pytest
import torch

import helpers as H
import helpers as H_mod  # (tests that use H for a height)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ext():
    from mappedconvolutions_b200 import host
    assert host.COMPILED, "extension not built: python -m mappedconvolutions_b200.build"
    return host.impl


def _cl(t):
    return t.contiguous(memory_format=torch.channels_last)


def _case(dtype, B, Cin, Cout, IH, IW, OH, OW, K, seed):
    g = torch.Generator().manual_seed(seed)
    c = lambda t: t.to(dtype).cuda()
    x, gy = c(torch.randn(B, Cin, IH, IW, generator=g)), c(torch.randn(B, Cout, OH, OW, generator=g))
    w, b = c(torch.randn(Cout, Cin, K, generator=g)), c(torch.randn(Cout, generator=g))
    m = (torch.rand(OH, OW, K, 2, generator=g) * torch.tensor([IW + 1.0, IH + 1.0]) - 1.0)
    m = m.to(torch.float64 if dtype == torch.float64 else torch.float32).cuda().contiguous()
    return x, gy, w, b, m


@pytest.mark.parametrize("dtype,layout,shape", [
    (torch.float32, "nchw", (2, 5, 7, 9, 11, 8, 10, 4)),
    (torch.float64, "nchw", (1, 3, 4, 6, 7, 5, 6, 3)),
    (torch.float32, "nhwc", (2, 8, 8, 9, 11, 8, 10, 4)),
    (torch.bfloat16, "nhwc", (2, 64, 128, 12, 20, 16, 32, 5)),   # tensor cores, plans cached
    (torch.bfloat16, "nchw", (2, 64, 64, 12, 20, 16, 32, 5)),    # rerouted through channels-last
])
@pytest.mark.parametrize("interp", [0, 1])
def test_conv_and_transposed_conv_match_the_ctypes_twin(ext, dtype, layout, shape, interp):
    from mappedconvolutions_b200 import ops
    B, Cin, Cout, IH, IW, OH, OW, K = shape
    x, gy, w, b, m = _case(dtype, *shape, seed=sum(shape) + interp)
    if layout == "nhwc":
        x, gy = _cl(x), _cl(gy)
    tol = H.TOL[dtype]
    for _ in range(2):  # the second round runs on cached plans
        y0, y1 = ops.mapped_conv_forward(x, m, w, b, K, interp), ext.mapped_conv_forward(x, m, w, b, K, interp)
        assert torch.equal(y0, y1) and y0.stride() == y1.stride()
        g0 = ops.mapped_conv_backward(gy, m, x, w, b, K, interp)
        g1 = ext.mapped_conv_backward(gy, m, x, w, b, K, interp)
        for a, c in zip(g0, g1):
            assert a.dtype == c.dtype and a.shape == c.shape
            H.assert_close(c.float(), a.float(), tol, "conv backward")
    assert ext.mapped_conv_backward(gy, m, x, w, b, K, interp, False)[0] is None
    # transposed layer: x plays grad_output's role
    wt = torch.randn(Cout, Cin, K, device="cuda").to(dtype)
    bt = torch.randn(Cin, device="cuda").to(dtype)
    t0 = ops.mapped_transposed_conv_forward(gy, m, wt, bt, IH, IW, K, interp)
    t1 = ext.mapped_transposed_conv_forward(gy, m, wt, bt, IH, IW, K, interp)
    H.assert_close(t1.float(), t0.float(), tol, "tconv forward")
    b0 = ops.mapped_transposed_conv_backward(x, m, gy, wt, bt, K, interp)
    b1 = ext.mapped_transposed_conv_backward(x, m, gy, wt, bt, K, interp)
    for a, c in zip(b0, b1):
        H.assert_close(c.float(), a.float(), tol, "tconv backward")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
def test_pool_resample_knn_match_the_ctypes_twin(ext, dtype, layout):
    from mappedconvolutions_b200 import ops
    g = torch.Generator().manual_seed(9)
    B, C, IH, IW, OH, OW, K = 2, 8, 10, 14, 6, 9, 7
    x = torch.randn(B, C, IH, IW, generator=g).to(dtype).cuda()
    gy = torch.randn(B, C, OH, OW, generator=g).to(dtype).cuda()
    if layout == "nhwc":
        x, gy = _cl(x), _cl(gy)
    m = (torch.rand(OH, OW, K, 2, generator=g) * torch.tensor([IW - 1.0, IH - 1.0])).cuda().contiguous()
    tol = H.TOL[dtype]
    for interp in (0, 1):
        y0, i0 = ops.mapped_max_pool(x, m, K, interp)
        y1, i1 = ext.mapped_max_pool(x, m, K, interp)
        assert torch.equal(y0, y1) and torch.equal(i0, i1)
        assert torch.equal(ops.mapped_avg_pool(x, m, K, interp), ext.mapped_avg_pool(x, m, K, interp))
        H.assert_close(ext.mapped_max_unpool(gy, i1, m, IH, IW, K, interp).float(),
                       ops.mapped_max_unpool(gy, i0, m, IH, IW, K, interp).float(), tol, "max unpool")
        H.assert_close(ext.mapped_avg_unpool(gy, m, IH, IW, K, interp).float(),
                       ops.mapped_avg_unpool(gy, m, IH, IW, K, interp).float(), tol, "avg unpool")
        m1 = m[:, :, :1, :].squeeze(2).contiguous()          # (OH, OW, 2) resample map
        assert torch.equal(ops.resample_from_map(x, m1, interp), ext.resample_from_map(x, m1, interp))
        H.assert_close(ext.resample_to_map(gy, m1, IH, IW, interp).float(),
                       ops.resample_to_map(gy, m1, IH, IW, interp).float(), tol, "resample_to_map")
    if dtype == torch.float32 and layout == "nchw":
        p = torch.randn(1, 3, 500, generator=g).cuda()
        a, c = ops.knn_forward(p, p, 5), ext.knn_forward(p, p, 5)
        assert torch.equal(a[0], c[0]) and torch.equal(a[1], c[1])


def test_errors_are_raised_like_in_the_ctypes_twin(ext):
    x = torch.zeros(1, 4, 4, 4)
    m = torch.zeros(4, 4, 1, 2)
    with pytest.raises(RuntimeError, match="CUDA only"):
        ext.mapped_avg_pool(x, m, 1, 0)
    with pytest.raises(RuntimeError, match="sample map"):
        ext.mapped_avg_pool(x.cuda(), m.double().cuda(), 1, 0)
    with pytest.raises(RuntimeError, match="contiguous"):
        ext.mapped_avg_pool(x.cuda().transpose(2, 3), m.cuda(), 1, 0)


def test_fused_relu_equals_conv_then_relu(ext):
    """activation='relu' runs max(0, .) in the convolution kernel's epilogue (MC_FLAG_RELU).  The
    result must equal relu(conv(x)) bit for bit - the clamp acts on the same float32 accumulator
    before the same rounding - and so must the input gradient."""
    from mapped_convolution.nn import MappedConvolution
    torch.manual_seed(11)
    for (B, Cin, Cout, Hh, Ww, K, interp, dt, cl) in (
            (2, 64, 64, 16, 32, 9, 1, torch.bfloat16, True),      # tensor-core kernel
            (1, 64, 128, 1, 642, 7, 0, torch.bfloat16, True),     # nearest map on a mesh
            (2, 5, 7, 9, 11, 4, 1, torch.float32, False)):        # generic kernel
        name = {0: "nearest", 1: "bilinear"}[interp]
        plain = MappedConvolution(Cin, Cout, K, name).cuda().to(dt)
        fused = MappedConvolution(Cin, Cout, K, name, activation="relu").cuda().to(dt)
        fused.load_state_dict(plain.state_dict())
        x = torch.randn(B, Cin, Hh, Ww, device="cuda").to(dt)
        if cl:
            x = x.contiguous(memory_format=torch.channels_last)
        m = (torch.rand(Hh, Ww, K, 2, device="cuda") * torch.tensor([Ww - 1.0, Hh - 1.0], device="cuda")).contiguous()
        xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
        ya = torch.relu(plain(xa, m))
        yb = fused(xb, m)
        assert torch.equal(ya, yb) and (yb >= 0).all() and (yb == 0).any()
        g = torch.randn_like(ya)
        ya.backward(g)
        yb.backward(g)
        # (the general weight-gradient kernels and the generic input-gradient kernel add partial sums
        # with atomics: two runs agree to rounding, not bit for bit)
        tol = 2e-2 if dt == torch.bfloat16 else 1e-5
        if dt == torch.bfloat16:
            assert torch.equal(xa.grad, xb.grad)
        else:
            H.assert_close(xb.grad, xa.grad, tol, "grad_x")
        H.assert_close(fused.weight.grad.float(), plain.weight.grad.float(), tol, "grad_w")
        H.assert_close(fused.bias.grad.float(), plain.bias.grad.float(), tol, "grad_b")


def test_row_plans_through_the_layer_api(ext):
    """A spherical (gnomonic) map on an equirectangular image is translation invariant along rows:
    the layer takes the row-plan kernels for forward, input gradient and weight gradient.  Results
    against the oracle (2e-2) and against the general kernels of the same library (row plans off)."""
    from mapped_convolution.nn import MappedConvolution
    from mapped_convolution.util import get_projection_map
    from oracle import oracle
    torch.manual_seed(12)
    Hh, Ww, C, K, B = 32, 512, 64, 9, 2
    m = get_projection_map((Hh, Ww), (3, 3), "gnomonic").contiguous().cuda()
    layer = MappedConvolution(C, C, K, "bilinear").cuda().to(torch.bfloat16)
    x = torch.randn(B, C, Hh, Ww, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    g = torch.randn(B, C, Hh, Ww, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)

    def run():
        layer.zero_grad()
        xi = x.clone().requires_grad_(True)
        y = layer(xi, m)
        y.backward(g)
        return y.detach(), xi.grad, layer.weight.grad.clone(), layer.bias.grad.clone()

    n0 = ext.mapped_conv_forward  # (touch the binding so that a missing symbol fails here)
    assert n0 is not None
    fast = run()
    was = ext.set_row_plans(False)
    try:
        slow = run()
    finally:
        ext.set_row_plans(was)
    w, b = layer.weight.detach().float().cpu(), layer.bias.detach().float().cpu()
    want_y = oracle.mapped_conv_forward(x.float().cpu().contiguous(), m.cpu(), w, b, K, 1)
    want = oracle.mapped_conv_backward(g.float().cpu().contiguous(), m.cpu(), x.float().cpu().contiguous(), w, b, K, 1)
    for name, got, ref, other in (("y", fast[0], want_y, slow[0]), ("grad_x", fast[1], want[0], slow[1]),
                                  ("grad_w", fast[2], want[1], slow[2]), ("grad_b", fast[3], want[2], slow[3])):
        H.assert_close(got.float(), ref, 2e-2, "row plan " + name + " vs oracle")
        H.assert_close(other.float(), ref, 2e-2, "general " + name + " vs oracle")
    assert not torch.equal(fast[0], slow[0])   # two different kernels really ran


def _weighted_case(P, interp, shape, seed):
    """bf16 channels-last tensors and a weighted map: P points per tap with positive weights that
    sum to one (barycentric style); point coordinates include a few outside the image."""
    B, Cin, Cout, IH, IW, OH, OW, K = shape
    g = torch.Generator().manual_seed(seed)
    c = lambda t: _cl(t.to(torch.bfloat16).cuda())
    x, gy = c(torch.randn(B, Cin, IH, IW, generator=g)), c(torch.randn(B, Cout, OH, OW, generator=g))
    w = torch.randn(Cout, Cin, K, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(Cout, generator=g).to(torch.bfloat16).cuda()
    m = torch.rand(OH, OW, K, P, 2, generator=g) * torch.tensor([IW + 1.0, IH + 1.0]) - 1.0
    if interp == 0:
        m = m.round()
    iw = torch.rand(OH, OW, K, P, generator=g) + 0.05
    iw = iw / iw.sum(-1, keepdim=True)
    iw[0, 0, 0, 0] = 0.0                                   # a point that contributes nothing
    return x, gy, w, b, m.float().cuda().contiguous(), iw.float().cuda().contiguous()


@pytest.mark.parametrize("name,P,interp,shape,kinds", [
    ("barycentric 64->128", 3, 0, (2, 64, 128, 1, 642, 1, 642, 7), {3, 4}),
    ("barycentric 64->64", 3, 0, (3, 64, 64, 1, 300, 1, 300, 7), {3, 4}),
    ("four points", 4, 0, (1, 128, 64, 12, 20, 16, 32, 5), {3, 4}),
    ("one bilinear point", 1, 1, (2, 64, 64, 12, 20, 16, 32, 4), {3, 4}),
    ("first layer 3->64", 3, 0, (2, 3, 64, 1, 642, 1, 642, 7), {4}),
    ("three bilinear points: does not fold", 3, 1, (1, 64, 64, 12, 20, 16, 32, 3), set()),
])
def test_weighted_conv_on_the_tensor_cores(ext, name, P, interp, shape, kinds):
    """A weighted map whose points fit a tap-table record runs on the tensor-core kernels with plans
    built from (map, weights); the result is the reference's weighted convolution (oracle, fp32 on
    the bf16-rounded tensors) within the bf16 tolerance, and equals the generic kernels' within it."""
    from mappedconvolutions_b200 import ops
    from oracle import oracle
    B, Cin, Cout, IH, IW, OH, OW, K = shape
    x, gy, w, b, m, iw = _weighted_case(P, interp, shape, seed=sum(shape) + P)
    tol = H.TOL[torch.bfloat16]
    ext.clear_plan_cache()
    for _ in range(2):  # the second round runs on cached plans
        y = ext.weighted_mapped_conv_forward(x, m, iw, w, b, K, interp)
        g = ext.weighted_mapped_conv_backward(gy, m, iw, x, w, b, K, interp)
    assert set(ext.plan_cache_kinds()) == kinds, name
    assert ext.device_status() == 0
    cpu = lambda t: t.float().cpu().contiguous()
    y_ref = oracle.weighted_mapped_conv_forward(cpu(x), m.cpu(), iw.cpu(), cpu(w), cpu(b), K, interp)
    g_ref = oracle.weighted_mapped_conv_backward(cpu(gy), m.cpu(), iw.cpu(), cpu(x), cpu(w), cpu(b), K, interp)
    H.assert_close(cpu(y), y_ref, tol, name + " forward")
    for got, want, what in zip(g, g_ref, ("grad_input", "grad_weight", "grad_bias")):
        H.assert_close(cpu(got), want, tol, name + " " + what)
    y_gen = ops.weighted_mapped_conv_forward(x, m, iw, w, b, K, interp)
    H.assert_close(cpu(y), cpu(y_gen), tol, name + " forward vs generic kernels")
    # the map tensor alone does not identify the plan: other weights, other result
    iw2 = (iw.flip(-1) if P > 1 else iw * 0.5).contiguous()
    y2 = ext.weighted_mapped_conv_forward(x, m, iw2, w, b, K, interp)
    y2_ref = oracle.weighted_mapped_conv_forward(cpu(x), m.cpu(), iw2.cpu(), cpu(w), cpu(b), K, interp)
    H.assert_close(cpu(y2), y2_ref, tol, name + " forward with other weights")
    # NCHW activations are rerouted through channels-last and come back in NCHW
    y_nchw = ext.weighted_mapped_conv_forward(x.contiguous(), m, iw, w, b, K, interp)
    assert y_nchw.is_contiguous()
    H.assert_close(cpu(y_nchw), y_ref, tol, name + " forward from NCHW")


@pytest.mark.parametrize("name,P,interp,shape,kinds", [
    ("barycentric 64->128", 3, 0, (2, 64, 128, 1, 300, 1, 642, 7), {3, 4}),
    ("two points 128->64", 2, 0, (1, 128, 64, 12, 20, 16, 32, 5), {3, 4}),
    ("three bilinear points: does not fold", 3, 1, (1, 64, 64, 12, 20, 16, 32, 3), set()),
])
def test_weighted_transposed_conv_on_the_tensor_cores(ext, name, P, interp, shape, kinds):
    """The transposed layer with a weighted map: x (B, Cin, H, W) lives on the map grid, the map points
    into the (OH, OW) result; same plans as the weighted convolution, roles swapped."""
    from oracle import oracle
    B, Cin, Cout, H, W, OH, OW, K = shape
    g = torch.Generator().manual_seed(sum(shape) + 7 * P)
    c = lambda t: _cl(t.to(torch.bfloat16).cuda())
    x, gy = c(torch.randn(B, Cin, H, W, generator=g)), c(torch.randn(B, Cout, OH, OW, generator=g))
    w = torch.randn(Cin, Cout, K, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(Cout, generator=g).to(torch.bfloat16).cuda()
    m = torch.rand(H, W, K, P, 2, generator=g) * torch.tensor([OW + 1.0, OH + 1.0]) - 1.0
    m = (m.round() if interp == 0 else m).float().cuda().contiguous()
    iw = torch.rand(H, W, K, P, generator=g) + 0.05
    iw = (iw / iw.sum(-1, keepdim=True)).float().cuda().contiguous()
    tol = H_mod.TOL[torch.bfloat16]
    ext.clear_plan_cache()
    for _ in range(2):
        y = ext.weighted_mapped_transposed_conv_forward(x, m, iw, w, b, OH, OW, K, interp)
        gr = ext.weighted_mapped_transposed_conv_backward(gy, m, iw, x, w, b, K, interp)
    assert set(ext.plan_cache_kinds()) == kinds, name
    assert ext.device_status() == 0
    cpu = lambda t: t.float().cpu().contiguous()
    y_ref = oracle.weighted_mapped_transposed_conv_forward(cpu(x), m.cpu(), iw.cpu(), cpu(w), cpu(b), OH, OW, K,
                                                           interp)
    g_ref = oracle.weighted_mapped_transposed_conv_backward(cpu(gy), m.cpu(), iw.cpu(), cpu(x), cpu(w), cpu(b), K,
                                                            interp)
    H_mod.assert_close(cpu(y), y_ref, tol, name + " forward")
    for got, want, what in zip(gr, g_ref, ("grad_input", "grad_weight", "grad_bias")):
        H_mod.assert_close(cpu(got), want, tol, name + " " + what)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("P,interp,folds", [(3, 0, True), (1, 1, True), (3, 1, False)])
def test_weighted_scatters_through_the_inverse_map(ext, dtype, P, interp, folds):
    """Weighted average unpooling and weighted resample-to-map: a weighted map whose points fit the
    inverse map's records is gathered through it (no atomics: the result repeats bit for bit), any
    other weighted map takes the atomic scatter; both agree with the oracle."""
    from oracle import oracle
    B, C, IH, IW, OH, OW, K = 2, 8, 13, 21, 10, 17, 4
    g = torch.Generator().manual_seed(100 * P + interp)
    gy = torch.randn(B, C, OH, OW, generator=g).to(dtype).cuda()
    m = torch.rand(OH, OW, K, P, 2, generator=g) * torch.tensor([IW + 1.0, IH + 1.0]) - 1.0
    m = (m.round() if interp == 0 else m).float().cuda().contiguous()
    iw = torch.rand(OH, OW, K, P, generator=g) + 0.05
    iw = (iw / iw.sum(-1, keepdim=True)).float().cuda().contiguous()
    tol = H_mod.TOL[dtype]
    cpu = lambda t: t.float().cpu().contiguous()
    ext.clear_plan_cache()
    gx = ext.weighted_mapped_avg_unpool(gy, m, iw, IH, IW, K, interp)
    assert (3 in ext.plan_cache_kinds()) == folds
    H_mod.assert_close(cpu(gx), oracle.weighted_mapped_avg_unpool(cpu(gy), m.cpu(), iw.cpu(), IH, IW, K, interp), tol,
                       "weighted avg unpool")
    if folds:
        assert torch.equal(gx, ext.weighted_mapped_avg_unpool(gy, m, iw, IH, IW, K, interp))
    # resample: one tap per grid pixel
    m1, iw1 = m[:, :, 0].contiguous(), iw[:, :, 0].contiguous()
    iw1 = (iw1 / iw1.sum(-1, keepdim=True)).contiguous()
    ext.clear_plan_cache()
    y = ext.weighted_resample_to_map(gy, m1, iw1, IH, IW, interp)
    assert (3 in ext.plan_cache_kinds()) == folds
    H_mod.assert_close(cpu(y), oracle.weighted_resample_to_map(cpu(gy), m1.cpu(), iw1.cpu(), IH, IW, interp), tol,
                       "weighted resample to map")
    if folds:
        assert torch.equal(y, ext.weighted_resample_to_map(gy, m1, iw1, IH, IW, interp))


@pytest.mark.parametrize("Cin,K,Cout,B,OHW,IHW", [
    (3, 7, 64, 5, (1, 333), (1, 333)),      # three n-tiles; images that end inside a 16-pixel step
    (1, 9, 64, 3, (6, 11), (7, 9)),         # two n-tiles, a 2-D image, taps outside the image
    (4, 7, 128, 2, (1, 100), (1, 50)),      # four n-tiles, two blocks of output channels
    (2, 3, 64, 1, (1, 16), (1, 16)),        # one n-tile, one step
    (3, 10, 64, 4, (1, 70), (1, 90)),       # 31 columns: the widest this kernel takes
])
def test_weight_gradient_of_layers_with_very_few_input_channels(ext, Cin, K, Cout, B, OHW, IHW):
    """Nearest maps, K * C_in + 1 <= 32: the weight / bias gradient runs in one pass over grad_output
    on warp-level MMAs (conv_wgrad_smallcin_kernel); against the oracle, fp32 on the bf16 tensors."""
    from oracle import oracle
    (OH, OW), (IH, IW) = OHW, IHW
    g = torch.Generator().manual_seed(Cin * 100 + K)
    c = lambda t: _cl(t.to(torch.bfloat16).cuda())
    x, gy = c(torch.randn(B, Cin, IH, IW, generator=g)), c(torch.randn(B, Cout, OH, OW, generator=g))
    w = torch.randn(Cout, Cin, K, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(Cout, generator=g).to(torch.bfloat16).cuda()
    m = (torch.rand(OH, OW, K, 2, generator=g) * torch.tensor([IW + 1.0, IH + 1.0]) - 1.0).round()
    m = m.float().cuda().contiguous()
    gr = ext.mapped_conv_backward(gy, m, x, w, b, K, 0)
    assert ext.device_status() == 0
    cpu = lambda t: t.float().cpu().contiguous()
    want = oracle.mapped_conv_backward(cpu(gy), m.cpu(), cpu(x), cpu(w), cpu(b), K, 0)
    for got, ref, what in zip(gr, want, ("grad_input", "grad_weight", "grad_bias")):
        H_mod.assert_close(cpu(got), ref, H_mod.TOL[torch.bfloat16], what)


def test_relu_gradient_inside_the_first_layer_weight_gradient(ext):
    """mapped_conv_backward(relu_output=y): grad_output counts where y > 0.  For a first layer (no input
    gradient, very few input channels) the weight-gradient kernel masks the rows as it loads them;
    everywhere else the op masks first.  Both must equal masking by hand."""
    g = torch.Generator().manual_seed(5)
    c = lambda t: _cl(t.to(torch.bfloat16).cuda())
    for Cin, Cout, K, n, need_gx in ((3, 64, 7, 1000, False), (3, 64, 7, 1000, True), (64, 64, 7, 300, False)):
        x, gy = c(torch.randn(3, Cin, 1, n, generator=g)), c(torch.randn(3, Cout, 1, n, generator=g))
        w = torch.randn(Cout, Cin, K, generator=g).to(torch.bfloat16).cuda()
        b = torch.randn(Cout, generator=g).to(torch.bfloat16).cuda()
        m = torch.zeros(1, n, K, 2)
        m[..., 0] = torch.randint(0, n, (1, n, K), generator=g).float()
        m = m.cuda()
        y = ext.mapped_conv_forward(x, m, w, b, K, 0, relu=True)
        assert 0.2 < (y > 0).float().mean().item() < 0.8
        got = ext.mapped_conv_backward(gy, m, x, w, b, K, 0, need_input_grad=need_gx, relu_output=y)
        want = ext.mapped_conv_backward(torch.ops.aten.threshold_backward(gy, y, 0), m, x, w, b, K, 0,
                                        need_input_grad=need_gx)
        assert (got[0] is None) == (not need_gx)
        for a, r, what in zip(got, want, ("grad_input", "grad_weight", "grad_bias")):
            if a is not None:
                H_mod.assert_close(a.float(), r.float(), H_mod.TOL[torch.bfloat16], what)
    assert ext.device_status() == 0
