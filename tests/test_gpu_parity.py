"""GPU parity tests proper: the CUDA path, called through the C-ABI, against the golden vectors of
the reference's CPU code and against the oracle on seeded inputs.

Bars: integer outputs (max-pool tap offsets, k-NN indices) bit-exact; gather-type float outputs
bit-exact as well (their arithmetic has no reordering freedom); everything that goes through a
contraction or an atomic accumulation within 1e-5 (float32), 1e-12 (float64), 2e-2 (bfloat16),
relative to max(|ref|, rms(ref))."""
import pytest
import torch

import helpers as H
from oracle import oracle

pytestmark = pytest.mark.gpu

RND = H.load_cases("random_small.npz")


def _impl(layout):
    from mappedconvolutions_b200 import ops
    return H.Impl(ops, "cuda", layout)


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
@pytest.mark.parametrize("name", sorted(n for n in RND if n.startswith("conv_")))
def test_conv_random(name, layout):
    c = RND[name]
    H.compare_case(H.run_conv(_impl(layout), c), c, H.TOL[c["input"].dtype], name)


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
@pytest.mark.parametrize("name", sorted(n for n in RND if n.startswith("tconv_")))
def test_tconv_random(name, layout):
    c = RND[name]
    H.compare_case(H.run_conv(_impl(layout), c, transposed=True), c, H.TOL[c["input"].dtype], name)


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
@pytest.mark.parametrize("name", sorted(n for n in RND if n.startswith("pool_f")))
def test_pool_random(name, layout):
    c = RND[name]
    H.compare_case(H.run_pool(_impl(layout), c), c, H.TOL[c["input"].dtype], name)


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
@pytest.mark.parametrize("name", sorted(n for n in RND if n.startswith("resample_")))
def test_resample_random(name, layout):
    c = RND[name]
    H.compare_case(H.run_resample(_impl(layout), c), c, H.TOL[c["input"].dtype], name)


def test_max_pool_uses_the_cuda_start_value():
    """All-negative windows return their true maximum and tap offset (the reference's CUDA build,
    include/nn/common/mapped_max_pool.h:29), not the CPU build's placeholder with index -1."""
    from mappedconvolutions_b200 import ops
    c = RND["pool_cpu_init_f32"]
    y, idx = ops.mapped_max_pool(c["input"].cuda(), c["sample_map"].cuda(), c["K"], c["interp"])
    y2, idx2 = oracle.mapped_max_pool(c["input"], c["sample_map"], c["K"], c["interp"], cuda_init=True)
    assert torch.equal(y.cpu(), y2) and torch.equal(idx.cpu(), idx2)
    ok = c["max_idx"] >= 0
    assert torch.equal(y.cpu()[ok], c["max_output"][ok]) and torch.equal(idx.cpu()[ok], c["max_idx"][ok])


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
def test_config1_float32(layout):
    c = H.load_cases("config1.npz")["config1"]
    H.compare_case(H.run_conv(_impl(layout), c), c, 1e-5, "config1")


# ---- seeded cases against the oracle -----------------------------------------------------------

def _one_ring_like_map(n_out, n_in, K, gen):
    """Nearest-mode map on an H = 1 image: tap 0 is the vertex itself, the others random vertices
    (with one duplicated tap per row now and then, as at an icosphere's valence-5 vertices)."""
    xs = torch.randint(0, n_in, (1, n_out, K), generator=gen).float()
    xs[0, :, 0] = torch.arange(n_out).float()
    dup = torch.rand(n_out, generator=gen) < 0.05
    xs[0, dup, K - 1] = xs[0, dup, 1]
    return torch.stack([xs, torch.zeros_like(xs)], -1).contiguous()


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
def test_pool_vertex_domain_bit_exact(layout):
    g = torch.Generator().manual_seed(7)
    B, C, Vin, Vout, K = 3, 16, 2562, 642, 7
    x = torch.randn(B, C, 1, Vin, generator=g)
    m = _one_ring_like_map(Vout, Vin, K, g)
    impl = _impl(layout)
    o = impl.ops
    y, idx = o.mapped_max_pool(impl.act(x), m.cuda(), K, 0)
    y2, idx2 = oracle.mapped_max_pool(x, m, K, 0, cuda_init=True)
    assert torch.equal(idx.cpu(), idx2) and torch.equal(y.cpu().contiguous(), y2)
    a = o.mapped_avg_pool(impl.act(x), m.cuda(), K, 0)
    assert torch.equal(a.cpu().contiguous(), oracle.mapped_avg_pool(x, m, K, 0))
    gy = torch.randn(B, C, 1, Vout, generator=g)
    H.assert_close(o.mapped_max_unpool(impl.act(gy), idx, m.cuda(), 1, Vin, K, 0),
                   oracle.mapped_max_unpool(gy, idx2, m, 1, Vin, K, 0), 1e-5, "max_unpool")
    H.assert_close(o.mapped_avg_unpool(impl.act(gy), m.cuda(), 1, Vin, K, 0),
                   oracle.mapped_avg_unpool(gy, m, 1, Vin, K, 0), 1e-5, "avg_unpool")


@pytest.mark.parametrize("interp", [0, 1, 2])
def test_bf16_conv_against_oracle_on_rounded_inputs(interp):
    """bfloat16 has no counterpart in the reference: the oracle runs in float32 on the
    bfloat16-rounded inputs; tolerance 2e-2."""
    from mappedconvolutions_b200 import ops
    g = torch.Generator().manual_seed(11)
    B, Cin, Cout, IH, IW, OH, OW, K = 2, 16, 24, 12, 20, 10, 18, 5
    bf = lambda t: t.to(torch.bfloat16)
    x, w, b = bf(torch.randn(B, Cin, IH, IW, generator=g)), bf(torch.randn(Cout, Cin, K, generator=g)), \
        bf(torch.randn(Cout, generator=g))
    gy = bf(torch.randn(B, Cout, OH, OW, generator=g))
    m = (torch.rand(OH, OW, K, 2, generator=g) * torch.tensor([IW + 1.0, IH + 1.0]) - 1.0).contiguous()
    want_y = oracle.mapped_conv_forward(x.float(), m, w.float(), b.float(), K, interp)
    want_g = oracle.mapped_conv_backward(gy.float(), m, x.float(), w.float(), b.float(), K, interp)
    for layout in ("nchw", "nhwc"):
        impl = H.Impl(ops, "cuda", layout)
        y = ops.mapped_conv_forward(impl.act(x), m.cuda(), w.cuda(), b.cuda(), K, interp)
        gx, gw, gb = ops.mapped_conv_backward(impl.act(gy), m.cuda(), impl.act(x), w.cuda(), b.cuda(),
                                              K, interp)
        assert y.dtype == torch.bfloat16 and gx.dtype == torch.bfloat16
        H.assert_close(y.float(), want_y, 2e-2, "bf16 y")
        H.assert_close(gx.float(), want_g[0], 2e-2, "bf16 gx")
        H.assert_close(gw.float(), want_g[1], 2e-2, "bf16 gw")
        H.assert_close(gb.float(), want_g[2], 2e-2, "bf16 gb")


def _device_status():
    from mappedconvolutions_b200 import _lib
    return _lib.lib().mc_device_status(torch.cuda.current_stream().cuda_stream, 1)


@pytest.mark.parametrize("shape", [
    # B, Cin, Cout, IH, IW, OH, OW, K : 2-D pixel tiles; one ragged linear tile; many tiles per SM
    (2, 64, 64, 16, 32, 16, 32, 9),
    (1, 64, 64, 11, 13, 9, 7, 4),
    (3, 128, 64, 20, 24, 24, 48, 3),
    (2, 64, 64, 1, 2562, 1, 642, 7),
    (4, 64, 64, 64, 128, 64, 128, 9),
    # wider layers: 128 / 256 output channels per CTA, weight slices streamed beside the stages,
    # several output-channel chunks (192 = 3 x 64, 512 = 2 x 256)
    (2, 64, 128, 1, 642, 1, 642, 7),
    (1, 128, 256, 1, 300, 1, 300, 7),
    (1, 256, 256, 1, 200, 1, 162, 7),
    (1, 64, 192, 8, 16, 8, 16, 3),
    (1, 64, 512, 8, 16, 8, 16, 2),
    # input channels that are not a multiple of 64: slices hold (tap, channel) elements of several
    # taps; 16-byte gathers when C_in % 8 == 0, element-wise otherwise (a 3-channel first layer)
    (2, 3, 64, 1, 642, 1, 642, 7),
    (1, 16, 64, 12, 20, 10, 18, 9),
    (1, 96, 128, 12, 20, 10, 18, 3),
    (1, 20, 64, 9, 9, 9, 9, 5),
    # K * C_in <= 64: one slice per tile, built row-per-thread from the global tap table
    (1, 4, 128, 16, 32, 16, 32, 9),
    (3, 3, 64, 5, 50, 5, 50, 9),
    # nearest maps of such layers read whole pixels (1, 3 or 4 channels) through the compact
    # table: an odd element count (the last word straddles the end of the tensor), one channel,
    # more taps than one pass of loads holds
    (1, 3, 64, 1, 643, 1, 643, 7),
    (2, 1, 64, 1, 333, 1, 333, 9),
    (1, 1, 64, 8, 16, 8, 16, 33),
    (1, 3, 64, 7, 9, 16, 16, 20),
    (2, 4, 64, 1, 500, 1, 700, 16),
])
@pytest.mark.parametrize("interp", [0, 1, 2])
def test_bf16_tensor_core_conv_forward(shape, interp):
    """The tcgen05 implicit-GEMM forward (bf16, channels-last, C_in % 64 == 0, C_out % 64 == 0)
    against the oracle run in float32 on the bf16-rounded inputs; tolerance 2e-2."""
    from mappedconvolutions_b200 import ops
    B, Cin, Cout, IH, IW, OH, OW, K = shape
    g = torch.Generator().manual_seed(sum(shape) + interp)
    bf = lambda t: t.to(torch.bfloat16)
    x = bf(torch.randn(B, Cin, IH, IW, generator=g))
    w = bf(torch.randn(Cout, Cin, K, generator=g))
    b = bf(torch.randn(Cout, generator=g))
    m = (torch.rand(OH, OW, K, 2, generator=g) * torch.tensor([IW + 1.0, IH + 1.0]) - 1.0).contiguous()
    if IH == 1:
        m[..., 1] = 0
    want = oracle.mapped_conv_forward(x.float(), m, w.float(), b.float(), K, interp)
    xd = x.cuda().contiguous(memory_format=torch.channels_last)
    y = ops.mapped_conv_forward(xd, m.cuda(), w.cuda(), b.cuda(), K, interp)
    assert _device_status() == 0
    # (a single-channel input is contiguous in both layouts and counts as NCHW: so does its result)
    assert y.dtype == torch.bfloat16
    assert y.is_contiguous() if Cin == 1 else y.is_contiguous(memory_format=torch.channels_last)
    H.assert_close(y.float(), want, 2e-2, "tc fwd")


@pytest.mark.parametrize("shape", [
    (2, 64, 64, 16, 32, 16, 32, 9),
    (1, 64, 64, 11, 13, 9, 7, 4),
    (3, 64, 64, 24, 48, 8, 16, 3),
    (2, 64, 64, 1, 2562, 1, 642, 7),
    (2, 64, 64, 64, 128, 64, 128, 9),
    # wider layers: the weight gradient is split into output-channel chunks and groups of
    # (tap, input channel) tiles; the input gradient streams its weight slices
    (2, 64, 128, 1, 642, 1, 642, 7),
    (1, 128, 64, 9, 14, 16, 32, 5),
    (1, 128, 256, 1, 300, 1, 300, 7),
    (1, 256, 256, 1, 200, 1, 162, 7),
    (1, 64, 192, 8, 16, 8, 16, 3),
    (1, 128, 512, 8, 16, 8, 16, 2),
    # C_in not a multiple of 64: weight gradient on the tensor cores, input gradient generic
    (2, 3, 64, 1, 642, 1, 642, 7),
    (1, 16, 64, 12, 20, 10, 18, 9),
    (1, 96, 128, 12, 20, 10, 18, 3),
    (1, 20, 64, 9, 9, 9, 9, 5),
    (1, 4, 128, 16, 32, 16, 32, 9),
    (3, 3, 64, 5, 50, 5, 50, 9),
    (1, 3, 64, 1, 643, 1, 643, 7),
    (2, 1, 64, 1, 333, 1, 333, 9),
    (1, 3, 64, 7, 9, 16, 16, 20),
    (2, 4, 64, 1, 500, 1, 700, 16),
])
@pytest.mark.parametrize("interp", [0, 1, 2])
def test_bf16_tensor_core_conv_backward(shape, interp):
    """Input gradient through the inverse map and weight / bias gradient on the tensor cores
    against the oracle in float32 on the bf16-rounded inputs (2e-2); the input gradient must also
    repeat bit for bit, since the gather form has no atomics."""
    from mappedconvolutions_b200 import ops
    B, Cin, Cout, IH, IW, OH, OW, K = shape
    g = torch.Generator().manual_seed(sum(shape) + 7 * interp)
    bf = lambda t: t.to(torch.bfloat16)
    x = bf(torch.randn(B, Cin, IH, IW, generator=g))
    gy = bf(torch.randn(B, Cout, OH, OW, generator=g))
    w = bf(torch.randn(Cout, Cin, K, generator=g))
    b = bf(torch.randn(Cout, generator=g))
    m = (torch.rand(OH, OW, K, 2, generator=g) * torch.tensor([IW + 1.0, IH + 1.0]) - 1.0).contiguous()
    if IH == 1:
        m[..., 1] = 0
    want = oracle.mapped_conv_backward(gy.float(), m, x.float(), w.float(), b.float(), K, interp)
    cl = lambda t: t.cuda().contiguous(memory_format=torch.channels_last)
    md = m.cuda()
    got = ops.mapped_conv_backward(cl(gy), md, cl(x), w.cuda(), b.cuda(), K, interp)
    assert _device_status() == 0
    H.assert_close(got[0].float(), want[0], 2e-2, "tc dgrad")
    H.assert_close(got[1].float(), want[1], 2e-2, "tc wgrad")
    H.assert_close(got[2].float(), want[2], 2e-2, "tc bias grad")
    if Cin % 64 == 0:
        again = ops.mapped_conv_backward(cl(gy), md, cl(x), w.cuda(), b.cuda(), K, interp)
        assert torch.equal(got[0], again[0])


@pytest.mark.parametrize("shape", [
    # B, Cin, Cout, H, W (layer input = map grid), OH, OW (layer output), K
    (2, 64, 64, 8, 16, 16, 32, 4),
    (1, 128, 64, 9, 14, 16, 32, 5),
    (1, 64, 128, 1, 300, 1, 642, 7),
    (1, 256, 128, 8, 16, 12, 20, 3),
])
@pytest.mark.parametrize("interp", [0, 1, 2])
def test_bf16_tensor_core_transposed_conv(shape, interp):
    """Transposed convolution on the tensor-core primitives (its forward is the gather-form input
    gradient of the equivalent convolution, its input gradient that convolution's forward, its
    weight gradient the same GEMM with the two tensors swapped) against the oracle in float32 on
    the bf16-rounded inputs; tolerance 2e-2."""
    from mappedconvolutions_b200 import ops
    B, Cin, Cout, Hh, Ww, OH, OW, K = shape
    g = torch.Generator().manual_seed(sum(shape) + 13 * interp)
    bf = lambda t: t.to(torch.bfloat16)
    x = bf(torch.randn(B, Cin, Hh, Ww, generator=g))
    gy = bf(torch.randn(B, Cout, OH, OW, generator=g))
    w = bf(torch.randn(Cin, Cout, K, generator=g))
    b = bf(torch.randn(Cout, generator=g))
    m = (torch.rand(Hh, Ww, K, 2, generator=g) * torch.tensor([OW + 1.0, OH + 1.0]) - 1.0).contiguous()
    if OH == 1:
        m[..., 1] = 0
    want_y = oracle.mapped_transposed_conv_forward(x.float(), m, w.float(), b.float(), OH, OW, K, interp)
    want_g = oracle.mapped_transposed_conv_backward(gy.float(), m, x.float(), w.float(), b.float(), K, interp)
    cl = lambda t: t.cuda().contiguous(memory_format=torch.channels_last)
    md = m.cuda()
    y = ops.mapped_transposed_conv_forward(cl(x), md, w.cuda(), b.cuda(), OH, OW, K, interp)
    got = ops.mapped_transposed_conv_backward(cl(gy), md, cl(x), w.cuda(), b.cuda(), K, interp)
    assert _device_status() == 0
    H.assert_close(y.float(), want_y, 2e-2, "tc tconv fwd")
    H.assert_close(got[0].float(), want_g[0], 2e-2, "tc tconv dgrad")
    H.assert_close(got[1].float(), want_g[1], 2e-2, "tc tconv wgrad")
    H.assert_close(got[2].float(), want_g[2], 2e-2, "tc tconv bias grad")


@pytest.mark.parametrize("shape", [
    # shapes whose forward needs the prebuilt tap table even when the caller brings only the map:
    # streamed weight slices (256 columns) and the one-slice row-per-thread producer
    (1, 128, 256, 1, 300, 1, 300, 7),
    (2, 3, 64, 6, 40, 6, 40, 9),
    (1, 64, 64, 16, 32, 16, 32, 9),
])
@pytest.mark.parametrize("interp", [0, 1])
def test_c_abi_forward_and_wgrad_with_a_bare_map(shape, interp):
    """mc_conv_fwd / mc_conv_wgrad called directly with the float map (no plan objects): the
    library builds what it needs inside the caller's workspace.  Against the oracle, 2e-2."""
    from mappedconvolutions_b200 import _lib
    L = _lib.lib()
    B, Cin, Cout, IH, IW, OH, OW, K = shape
    g = torch.Generator().manual_seed(sum(shape) + interp)
    bf = lambda t: t.to(torch.bfloat16)
    x = bf(torch.randn(B, Cin, IH, IW, generator=g))
    gy = bf(torch.randn(B, Cout, OH, OW, generator=g))
    w = bf(torch.randn(Cout, Cin, K, generator=g))
    b = bf(torch.randn(Cout, generator=g))
    m = (torch.rand(OH, OW, K, 2, generator=g) * torch.tensor([IW + 1.0, IH + 1.0]) - 1.0).contiguous()
    if IH == 1:
        m[..., 1] = 0
    want_y = oracle.mapped_conv_forward(x.float(), m, w.float(), b.float(), K, interp)
    want_g = oracle.mapped_conv_backward(gy.float(), m, x.float(), w.float(), b.float(), K, interp)
    cl = lambda t: t.cuda().contiguous(memory_format=torch.channels_last)
    xd, gd, wd, bd, md = cl(x), cl(gy), w.cuda(), b.cuda(), m.cuda()
    d = _lib.McDesc(B, Cin, Cout, IH, IW, OH, OW, K, 0, interp, _lib.MC_BF16, _lib.MC_NHWC)
    st = torch.cuda.current_stream().cuda_stream
    n = max(L.mc_conv_fwd_workspace_bytes(d), L.mc_conv_wgrad_workspace_bytes(d), 16)
    assert L.mc_conv_fwd_workspace_bytes(d) > 0, "expected the tensor-core forward for this shape"
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    y = torch.empty_like(gd)
    _lib.check(L.mc_conv_fwd(d, xd.data_ptr(), md.data_ptr(), None, wd.data_ptr(), bd.data_ptr(),
                             y.data_ptr(), ws.data_ptr(), n, st))
    gw = torch.empty(Cout, Cin, K, dtype=torch.float32, device="cuda")
    gb = torch.empty(Cout, dtype=torch.float32, device="cuda")
    _lib.check(L.mc_conv_wgrad(d, gd.data_ptr(), xd.data_ptr(), md.data_ptr(), None, gw.data_ptr(),
                               gb.data_ptr(), ws.data_ptr(), n, st))
    assert _device_status() == 0
    H.assert_close(y.float(), want_y, 2e-2, "mc_conv_fwd")
    H.assert_close(gw, want_g[1], 2e-2, "mc_conv_wgrad")
    H.assert_close(gb, want_g[2], 2e-2, "mc_conv_wgrad bias")


@pytest.mark.parametrize("interp", [0, 1])
def test_bf16_nchw_tensors_take_the_tensor_core_path_and_keep_their_layout(interp):
    """bfloat16 tensors in the reference's NCHW layout are rerouted through channels-last copies;
    results come back in NCHW and match the oracle (2e-2)."""
    from mappedconvolutions_b200 import ops, _lib
    B, Cin, Cout, IH, IW, OH, OW, K = 2, 64, 128, 12, 20, 16, 32, 5
    g = torch.Generator().manual_seed(77 + interp)
    bf = lambda t: t.to(torch.bfloat16)
    x = bf(torch.randn(B, Cin, IH, IW, generator=g))
    gy = bf(torch.randn(B, Cout, OH, OW, generator=g))
    w = bf(torch.randn(Cout, Cin, K, generator=g))
    b = bf(torch.randn(Cout, generator=g))
    m = (torch.rand(OH, OW, K, 2, generator=g) * torch.tensor([IW + 1.0, IH + 1.0]) - 1.0).contiguous()
    want_y = oracle.mapped_conv_forward(x.float(), m, w.float(), b.float(), K, interp)
    want_g = oracle.mapped_conv_backward(gy.float(), m, x.float(), w.float(), b.float(), K, interp)
    n0 = _lib.lib().mc_kernel_launch_count()
    y = ops.mapped_conv_forward(x.cuda(), m.cuda(), w.cuda(), b.cuda(), K, interp)
    got = ops.mapped_conv_backward(gy.cuda(), m.cuda(), x.cuda(), w.cuda(), b.cuda(), K, interp)
    assert _device_status() == 0
    assert y.is_contiguous() and got[0].is_contiguous()
    H.assert_close(y.float(), want_y, 2e-2, "nchw y")
    H.assert_close(got[0].float(), want_g[0], 2e-2, "nchw gx")
    H.assert_close(got[1].float(), want_g[1], 2e-2, "nchw gw")
    H.assert_close(got[2].float(), want_g[2], 2e-2, "nchw gb")
    # transposed layer, same tensors with the roles of the two images exchanged
    wt = bf(torch.randn(Cout, Cin, K, generator=g))      # (C_in of the layer = Cout here, C_out = Cin)
    bt = bf(torch.randn(Cin, generator=g))
    want_t = oracle.mapped_transposed_conv_forward(gy.float(), m, wt.float(), bt.float(), IH, IW, K, interp)
    yt = ops.mapped_transposed_conv_forward(gy.cuda(), m.cuda(), wt.cuda(), bt.cuda(), IH, IW, K, interp)
    assert yt.is_contiguous()
    H.assert_close(yt.float(), want_t, 2e-2, "nchw tconv y")
    want_tg = oracle.mapped_transposed_conv_backward(x.float(), m, gy.float(), wt.float(), bt.float(), K, interp)
    gt = ops.mapped_transposed_conv_backward(x.cuda(), m.cuda(), gy.cuda(), wt.cuda(), bt.cuda(), K, interp)
    assert gt[0].is_contiguous()
    for a, r, what in zip(gt, want_tg, ("gx", "gw", "gb")):
        H.assert_close(a.float(), r, 2e-2, "nchw tconv " + what)


def test_bias_grad_entry_point():
    """mc_bias_grad against a float64 sum, both layouts and all dtypes (1e-5 / 2e-2)."""
    from mappedconvolutions_b200 import _lib
    L = _lib.lib()
    g = torch.Generator().manual_seed(5)
    for dt, code, tol in ((torch.float32, _lib.MC_F32, 1e-5), (torch.float64, _lib.MC_F64, 1e-12),
                          (torch.bfloat16, _lib.MC_BF16, 2e-2)):
        for C in (6, 64, 200):
            gy = torch.randn(3, C, 7, 33, generator=g).to(dt).cuda()
            want = gy.double().sum((0, 2, 3))
            for layout, t in ((_lib.MC_NCHW, gy.contiguous()),
                              (_lib.MC_NHWC, gy.contiguous(memory_format=torch.channels_last))):
                gb = torch.empty(C, dtype=torch.float64 if dt == torch.float64 else torch.float32,
                                 device="cuda")
                d = _lib.McDesc(3, C, C, 7, 33, 7, 33, 1, 0, 0, code, layout)
                _lib.check(L.mc_bias_grad(d, t.data_ptr(), gb.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream))
                H.assert_close(gb.double().cpu(), want.cpu(), tol, "bias grad")


def test_bf16_pool_and_resample():
    from mappedconvolutions_b200 import ops
    g = torch.Generator().manual_seed(12)
    x = torch.randn(2, 8, 9, 11, generator=g).to(torch.bfloat16)
    m = (torch.rand(6, 7, 4, 2, generator=g) * torch.tensor([12.0, 10.0]) - 1.0).contiguous()
    y, idx = ops.mapped_max_pool(x.cuda(), m.cuda(), 4, 0)
    y2, idx2 = oracle.mapped_max_pool(x.float(), m, 4, 0, cuda_init=True)
    assert torch.equal(idx.cpu(), idx2) and torch.equal(y.float().cpu(), y2)
    a = ops.mapped_avg_pool(x.cuda(), m.cuda(), 4, 1)
    H.assert_close(a.float(), oracle.mapped_avg_pool(x.float(), m, 4, 1), 2e-2, "bf16 avg")
    gy = torch.randn(2, 8, 6, 7, generator=g).to(torch.bfloat16)
    u = ops.mapped_avg_unpool(gy.cuda(), m.cuda(), 9, 11, 4, 1)
    H.assert_close(u.float(), oracle.mapped_avg_unpool(gy.float(), m, 9, 11, 4, 1), 2e-2, "bf16 unpool")
    # channels-last, nearest and bilinear: the vectorised gathers through the inverse map
    cl = lambda t: t.cuda().contiguous(memory_format=torch.channels_last)
    gy = torch.randn(3, 64, 6, 7, generator=g).to(torch.bfloat16)
    img = torch.randn(3, 64, 9, 11, generator=g).to(torch.bfloat16)
    for interp in (0, 1):
        u = ops.mapped_avg_unpool(cl(gy), m.cuda(), 9, 11, 4, interp)
        assert u.is_contiguous(memory_format=torch.channels_last)
        H.assert_close(u.float(), oracle.mapped_avg_unpool(gy.float(), m, 9, 11, 4, interp), 2e-2,
                       "bf16 unpool, channels-last")
        m1 = m[:, :, :1].contiguous()
        r = ops.resample_to_map(cl(gy), m1.cuda(), 9, 11, interp)
        H.assert_close(r.float(), oracle.resample_to_map(gy.float(), m1, 9, 11, interp), 2e-2,
                       "bf16 resample scatter, channels-last")
        a = ops.mapped_avg_pool(cl(img), m.cuda(), 4, interp)
        H.assert_close(a.float(), oracle.mapped_avg_pool(img.float(), m, 4, interp), 2e-2,
                       "bf16 avg pool, channels-last")


def test_empty_and_degenerate_shapes():
    """Single pixel, single channel, K = 1, a map whose samples are all outside the image."""
    from mappedconvolutions_b200 import ops
    x = torch.randn(1, 1, 1, 1).cuda()
    m = torch.zeros(1, 1, 1, 2).cuda()
    w = torch.ones(1, 1, 1).cuda()
    b = torch.zeros(1).cuda()
    assert torch.equal(ops.mapped_conv_forward(x, m, w, b, 1, 1), x)
    far = torch.full((3, 3, 2, 2), 1e9).cuda()
    xx = torch.randn(2, 3, 4, 4).cuda()
    assert torch.count_nonzero(ops.mapped_avg_pool(xx, far, 2, 1)) == 0
    y, idx = ops.mapped_max_pool(xx, far, 2, 0)
    assert torch.count_nonzero(y) == 0 and (idx == torch.arange(9, device="cuda").view(3, 3) * 4).all()


def test_non_contiguous_input_is_rejected():
    from mappedconvolutions_b200 import ops
    x = torch.randn(2, 3, 4, 8).cuda()[..., ::2]
    with pytest.raises(RuntimeError):
        ops.mapped_avg_pool(x, torch.zeros(2, 2, 1, 2).cuda(), 1, 0)


# ---- k nearest neighbours ----------------------------------------------------------------------

@pytest.mark.parametrize("D,M,N,k", [(3, 2562, 2562, 9), (3, 700, 333, 1), (2, 1000, 50, 16),
                                     (5, 300, 257, 20), (3, 40, 40, 32), (16, 129, 65, 4)])
def test_knn_bit_exact_against_oracle(D, M, N, k):
    from mappedconvolutions_b200 import ops
    g = torch.Generator().manual_seed(D * 1000 + k)
    ref = torch.randn(2, D, M, generator=g)
    if D == 3:
        ref = ref / ref.norm(dim=1, keepdim=True)  # points on the unit sphere
        ref[:, :, 5] = ref[:, :, 3]                # exact duplicates: ties broken by index
    q = ref[:, :, :N].clone() if N <= M else torch.randn(2, D, N, generator=g)
    idx, dist = ops.knn_forward(ref.cuda(), q.cuda(), k)
    idx2, dist2 = oracle.knn_forward(ref, q, k)
    assert idx.dtype == torch.int64 and torch.equal(idx.cpu(), idx2)
    assert torch.equal(dist.cpu(), dist2)
    assert idx.min() >= 1 and idx.max() <= M


def test_knn_self_match_is_first_and_one_based():
    from mapped_convolution.util import knn
    g = torch.Generator().manual_seed(3)
    p = torch.randn(1, 3, 500, generator=g).cuda()
    idx, dist = knn(p, p, 4)
    assert torch.equal(idx[0, 0], torch.arange(1, 501, device="cuda"))
    assert torch.count_nonzero(dist[0, 0]) == 0
    assert (dist[0, 1:] >= dist[0, :-1]).all()


def test_a_bounded_wait_that_runs_out_is_reported_and_the_library_stays_usable(op_binding):
    """The tensor-core kernels never wait without a limit: a wait that runs out raises the block's
    abort flag and the device status word and the kernel returns.  mc_selftest_wait_expiry drives
    that path on purpose with a one-warp kernel waiting a millisecond on a barrier nobody arrives
    at; afterwards mc_device_status reports the code once, and ordinary calls work as before."""
    from mappedconvolutions_b200 import _lib, ops
    L = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    assert L.mc_device_status(st, 1) == 0
    seen = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(L.mc_selftest_wait_expiry(seen.data_ptr(), st))
    assert L.mc_device_status(st, 1) == 0x7F1        # raised by the wait; the read clears it
    assert seen.item() == 2                           # abort flag set, the wait returned false
    assert L.mc_device_status(st, 0) == 0
    g = torch.Generator().manual_seed(9)
    x = torch.randn(1, 64, 8, 16, generator=g).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
    m = (torch.rand(8, 16, 4, 2, generator=g) * torch.tensor([15., 7.])).cuda()
    w, b = torch.randn(64, 64, 4, generator=g).to(torch.bfloat16).cuda(), torch.zeros(64, dtype=torch.bfloat16).cuda()
    y = ops.mapped_conv_forward(x, m, w, b, 4, 1)
    want = oracle.mapped_conv_forward(x.float().cpu().contiguous(), m.cpu(), w.float().cpu(), b.float().cpu(), 4, 1)
    H.assert_close(y.float(), want, 2e-2, "forward after the self-test")
    assert L.mc_device_status(st, 1) == 0


def test_non_finite_input_next_to_a_tap_that_reads_nothing(op_binding):
    """Documented deviation of the bf16 tensor-core kernels: their tap records always point at real
    pixels (a corner that contributes nothing gets weight 0 and the address of a pixel the tap reads
    anyway, a tap that reads nothing at all the address of pixel 0), so that the gather needs no
    predicates.  The reference skips such corners (include/core/interpolation.h:125-154).  With
    finite inputs the two agree; a NaN in pixel 0 of an image reaches, through 0 * NaN, exactly the
    outputs that have a tap lying completely outside the image - and no others."""
    from mappedconvolutions_b200 import ops
    g = torch.Generator().manual_seed(10)
    Hh, Ww, K = 8, 16, 4
    x = torch.randn(1, 64, Hh, Ww, generator=g).to(torch.bfloat16)
    m = torch.rand(Hh, Ww, K, 2, generator=g) * torch.tensor([Ww - 3.0, Hh - 3.0]) + 1.0   # all inside,
    assert not ((m[..., 0] < 1) & (m[..., 1] < 1)).any()                                   # none reads pixel 0
    outside = torch.zeros(Hh, Ww, dtype=torch.bool)
    outside[2, 3] = outside[5, 9] = True
    m[outside, 1, :] = torch.tensor([-7.5, -3.25])          # tap 1 of two pixels reads nothing
    w, b = torch.randn(64, 64, K, generator=g).to(torch.bfloat16), torch.zeros(64, dtype=torch.bfloat16)
    cl = lambda t: t.cuda().contiguous(memory_format=torch.channels_last)
    clean = ops.mapped_conv_forward(cl(x), m.cuda(), w.cuda(), b.cuda(), K, 1)
    want = oracle.mapped_conv_forward(x.float(), m, w.float(), b.float(), K, 1)
    H.assert_close(clean.float(), want, 2e-2, "finite input")
    xn = x.clone()
    xn[0, :, 0, 0] = float("nan")
    y = ops.mapped_conv_forward(cl(xn), m.cuda(), w.cuda(), b.cuda(), K, 1)
    nan_at = torch.isnan(y.float()).any(1)[0].cpu()
    assert torch.equal(nan_at, outside)
    assert torch.equal(y[0][:, ~outside.cuda()], clean[0][:, ~outside.cuda()])


@pytest.mark.parametrize("name", sorted(H.load_cases("knn_ref.npz")))
def test_knn_equals_the_reference_cuda_kernels(name, op_binding):
    """mc_knn against outputs of the reference's own CUDA k-NN (include/util/cuda/knn.cuh:42-205)
    recorded on a B200 - indices and distances bit for bit, exact duplicates among the reference
    points and zero distances included."""
    from mappedconvolutions_b200 import ops
    c = H.load_cases("knn_ref.npz")[name]
    idx, dist = ops.knn_forward(c["ref"].cuda(), c["query"].cuda(), int(c["k"]))
    assert torch.equal(idx.cpu(), c["idx"])
    assert torch.equal(dist.cpu(), c["dist"])


def test_tensor_core_kernels_on_a_second_device(op_binding):
    """Shared-memory opt-in, SM count and the static scratch address are properties of a device, not
    of the process: after a call on device 0 the same process must be able to run the tensor-core
    kernels on device 1 (plain local kernels, no peer memory)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    from mappedconvolutions_b200 import ops
    g = torch.Generator().manual_seed(21)
    Hh, Ww, K = 8, 16, 4
    x = torch.randn(1, 64, Hh, Ww, generator=g).to(torch.bfloat16)
    m = torch.rand(Hh, Ww, K, 2, generator=g) * torch.tensor([Ww - 1.0, Hh - 1.0])
    w, b = torch.randn(64, 64, K, generator=g).to(torch.bfloat16), torch.randn(64, generator=g).to(torch.bfloat16)
    want = oracle.mapped_conv_forward(x.float(), m, w.float(), b.float(), K, 1)
    for dev in ("cuda:0", "cuda:1", "cuda:0"):
        with torch.cuda.device(dev):
            xd = x.to(dev).contiguous(memory_format=torch.channels_last)
            y = ops.mapped_conv_forward(xd, m.to(dev), w.to(dev), b.to(dev), K, 1)
            H.assert_close(y.float().cpu(), want, 2e-2, "forward on " + dev)


@pytest.mark.parametrize("interp", [0, 1])
def test_input_gradient_with_the_contraction_first(interp, op_binding):
    """Layers with more output than input channels take mc_conv_dgrad_tapsum: grad_output times the
    weights of every tap as one dense GEMM, then a gather-sum of the narrow rows through the inverse
    map.  Against the oracle, and against the gather-in-the-GEMM form (mc_conv_dgrad_inv) on the
    same inverse map."""
    from mappedconvolutions_b200 import _lib, ops
    L = _lib.lib()
    g = torch.Generator().manual_seed(31 + interp)
    B, Cin, Cout, Hh, Ww, K = 3, 64, 128, 9, 20, 5
    bf = torch.bfloat16
    x = torch.randn(B, Cin, Hh, Ww, generator=g).to(bf)
    gy = torch.randn(B, Cout, Hh, Ww, generator=g).to(bf)
    w, b = (torch.randn(Cout, Cin, K, generator=g) * 0.2).to(bf), torch.zeros(Cout).to(bf)
    m = torch.rand(Hh, Ww, K, 2, generator=g) * torch.tensor([Ww + 1.0, Hh + 1.0]) - 1.0   # some taps outside
    cl = lambda t: t.cuda().contiguous(memory_format=torch.channels_last)
    gx = ops.mapped_conv_backward(cl(gy), m.cuda(), cl(x), w.cuda(), b.cuda(), K, interp)[0]
    want = oracle.mapped_conv_backward(gy.float(), m, x.float(), w.float(), b.float(), K, interp)[0]
    H.assert_close(gx.float(), want, 2e-2, "grad_x, contraction first, vs oracle")
    import importlib
    pyops = importlib.import_module("mappedconvolutions_b200.ops")   # (the ctypes twin, for its helpers)
    d = _lib.McDesc(B, Cin, Cout, Hh, Ww, Hh, Ww, K, 0, interp, _lib.MC_BF16, _lib.MC_NHWC)
    assert pyops._contract_first(d)
    inv = pyops._inverse_map(d, m.cuda().contiguous())
    gx2 = torch.empty_like(gx)
    nws = L.mc_conv_dgrad_inv_workspace_bytes(d)
    ws = torch.empty(max(nws, 16), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(L.mc_conv_dgrad_inv(d, cl(gy).data_ptr(), inv.data_ptr(), w.cuda().data_ptr(), None,
                                   gx2.data_ptr(), ws.data_ptr(), nws, st))
    H.assert_close(gx.float(), gx2.float(), 2e-2, "grad_x, contraction first, vs gather in the GEMM")
