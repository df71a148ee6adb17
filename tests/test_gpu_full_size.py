"""The configurations of the headline benchmark at their FULL sizes, checked through properties that
do not need a CPU run of the whole workload:

* adjoint identities  <A x, g> == <x, A^T g>  tie a forward op to its backward op (every op on
  this path is linear in the tensor it gathers from, and the convolution also in its weights);
* batch independence: element b of a batch-B call equals the batch-1 call on that element (bit
  for bit where the kernel has no atomics), so that parity of ONE element against the oracle - which
  the oracle finishes in seconds - carries over to the whole batch;
* pooling against an independent formulation with torch indexing; k-NN through sortedness, the
  self match and recomputed distances, plus exact agreement with a brute-force search on a sample
  of the queries.

Inner products are accumulated in float64 and compared on the scale |a| |b| / sqrt(n) - the size
of an inner product of two unrelated vectors, which is what a wrong backward op would be off by:
2e-2 of it for bfloat16 ops (their outputs are rounded to 8 bits), 1e-4 for float32 ops.
Element-wise comparisons: float32 1e-5, bfloat16 2e-2."""
import pytest
import torch

import helpers as H
from oracle import oracle

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _dot(a, b):
    return (a.double() * b.double()).sum().item()


def _cl(t):
    return t.contiguous(memory_format=torch.channels_last)


def _assert_adjoint(a, b, a2, b2, tol, what):
    """<a, b> == <a2, b2> on the scale |a2| |b2| / sqrt(n)."""
    lhs, rhs = _dot(a, b), _dot(a2, b2)
    scale = a2.double().norm().item() * b2.double().norm().item() / a2.numel() ** 0.5
    assert abs(lhs - rhs) <= tol * scale, "%s: %r vs %r (scale %r)" % (what, lhs, rhs, scale)


@pytest.fixture(scope="module")
def config2():
    """Spherical conv, 512x1024, batch 8, 64 -> 64, gnomonic 3x3 map, bilinear, bf16."""
    from mappedconvolutions_b200.util import get_projection_map
    g = torch.Generator().manual_seed(2)
    B, C, Hh, Ww, K = 8, 64, 512, 1024, 9
    bf = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16)
    x, gy = _cl(bf(B, C, Hh, Ww).to(DEV)), _cl(bf(B, C, Hh, Ww).to(DEV))
    w, b = bf(C, C, K).to(DEV), bf(C).to(DEV)
    m = get_projection_map((Hh, Ww), (3, 3), "gnomonic").contiguous().to(DEV)
    return dict(x=x, gy=gy, w=w, b=b, m=m, K=K)


def test_config2_adjoint_identities(config2):
    from mappedconvolutions_b200 import ops
    c = config2
    x, gy, w, b, m, K = c["x"], c["gy"], c["w"], c["b"], c["m"], c["K"]
    zero_b = torch.zeros_like(b)
    y = ops.mapped_conv_forward(x, m, w, zero_b, K, 1)
    gx, gw, gb = ops.mapped_conv_backward(gy, m, x, w, b, K, 1)
    # forward and input gradient are adjoint in x; forward and weight gradient in w
    _assert_adjoint(y, gy, x, gx, 2e-2, "<y, gy> == <x, grad_x>")
    _assert_adjoint(y, gy, w, gw, 2e-2, "<y, gy> == <w, grad_w>")
    # bias gradient = sum of grad_output
    want_gb = gy.double().sum((0, 2, 3))
    H.assert_close(gb.double().cpu(), want_gb.cpu(), 2e-2, "grad_bias")
    # the bias enters the forward pass additively
    yb = ops.mapped_conv_forward(x, m, w, b, K, 1)
    d = (yb.float() - y.float()) - b.float().view(1, -1, 1, 1)
    assert d.abs().max().item() <= 2e-2 * (y.float().abs().max().item() + 1.0)


def test_config2_batch_independence_and_oracle_on_one_element(config2):
    from mappedconvolutions_b200 import ops
    c = config2
    x, gy, w, b, m, K = c["x"], c["gy"], c["w"], c["b"], c["m"], c["K"]
    y = ops.mapped_conv_forward(x, m, w, b, K, 1)
    gx, gw, gb = ops.mapped_conv_backward(gy, m, x, w, b, K, 1)
    for e in (0, 5):
        y1 = ops.mapped_conv_forward(_cl(x[e:e + 1]), m, w, b, K, 1)
        gx1, _, _ = ops.mapped_conv_backward(_cl(gy[e:e + 1]), m, _cl(x[e:e + 1]), w, b, K, 1)
        assert torch.equal(y1[0], y[e])      # no atomics in forward / input gradient:
        assert torch.equal(gx1[0], gx[e])    # bit for bit
    # weight gradient of the batch = sum of the per-element weight gradients
    acc = torch.zeros_like(gw, dtype=torch.float32)
    for e in range(x.shape[0]):
        acc += ops.mapped_conv_backward(_cl(gy[e:e + 1]), m, _cl(x[e:e + 1]), w, b, K, 1)[1].float()
    H.assert_close(gw.float(), acc, 2e-2, "grad_w batch sum")
    # element 3 against the oracle (float32 on the bf16-rounded inputs), full 512 x 1024 image
    e = 3
    xc, gc = x[e:e + 1].float().cpu().contiguous(), gy[e:e + 1].float().cpu().contiguous()
    want_y = oracle.mapped_conv_forward(xc, m.cpu(), w.float().cpu(), b.float().cpu(), K, 1)
    want_g = oracle.mapped_conv_backward(gc, m.cpu(), xc, w.float().cpu(), b.float().cpu(), K, 1)
    H.assert_close(y[e:e + 1].float(), want_y, 2e-2, "y vs oracle")
    H.assert_close(gx[e:e + 1].float(), want_g[0], 2e-2, "grad_x vs oracle")
    g1 = ops.mapped_conv_backward(_cl(gy[e:e + 1]), m, _cl(x[e:e + 1]), w, b, K, 1)
    H.assert_close(g1[1].float(), want_g[1], 2e-2, "grad_w vs oracle")
    H.assert_close(g1[2].float(), want_g[2], 2e-2, "grad_b vs oracle")


def test_config3_resample_adjoint_and_oracle():
    """Equirect 512x1024x3 float32, batch 16 <-> icosphere level-7 vertices, bilinear."""
    from mappedconvolutions_b200 import ops
    from mappedconvolutions_b200.util import icosphere as ico
    g = torch.Generator().manual_seed(3)
    img = torch.rand(16, 3, 512, 1024, generator=g)
    from mappedconvolutions_b200 import util as mutil
    m = mutil.image_to_sphere_resample_map((512, 1024), mutil.generate_icosphere(7))
    v = torch.rand(16, 3, m.shape[0], m.shape[1], generator=g)
    imgd, md, vd = img.to(DEV), m.to(DEV), v.to(DEV)
    gathered = ops.resample_from_map(imgd, md, 1)
    scattered = ops.resample_to_map(vd, md, 512, 1024, 1)
    _assert_adjoint(gathered, vd, imgd, scattered, 1e-4, "resample gather / scatter")
    # two batch elements against the oracle: the gather is bit exact, the scatter-add 1e-5
    want_g = oracle.resample_from_map(img[4:6].contiguous(), m, 1)
    assert torch.equal(gathered[4:6].cpu(), want_g)
    want_s = oracle.resample_to_map(v[4:6].contiguous(), m, 512, 1024, 1)
    H.assert_close(scattered[4:6], want_s, 1e-5, "resample_to_map")


def _torch_pool_taps(x, m):
    """(B, C, N_out, K) tap values of a nearest-interpolation vertex map, by torch indexing."""
    idx = torch.round(m[0, :, :, 0]).long()          # (N_out, K) vertex indices (y is 0)
    return x[:, :, 0, :][:, :, idx]


def test_config4_pooling_against_torch_indexing():
    """Icosphere level 7 -> 6, 7-tap one-ring, nearest, batch 32, 128 channels, float32."""
    from mappedconvolutions_b200 import ops
    from mappedconvolutions_b200.util import icosphere as ico
    g = torch.Generator().manual_seed(4)
    x = torch.randn(32, 128, 1, ico.num_vertices(7), generator=g).to(DEV)
    m = ico.pooling_map(7).to(DEV)
    taps = _torch_pool_taps(x, m)
    ymax, idx = ops.mapped_max_pool(x, m, 7, 0)
    assert torch.equal(ymax[:, :, 0, :], taps.max(dim=3).values)
    # the stored offsets point at a tap that holds the maximum: offset = (vertex * K + tap) * 2
    tap = (idx[:, :, 0, :] // 2) % 7
    vert = (idx[:, :, 0, :] // 2) // 7
    assert torch.equal(vert, torch.arange(m.shape[1], device=DEV).expand_as(vert))
    assert torch.equal(taps.gather(3, tap.unsqueeze(3)).squeeze(3), ymax[:, :, 0, :])
    yavg = ops.mapped_avg_pool(x, m, 7, 0)
    H.assert_close(yavg[:, :, 0, :], taps.double().sum(3).float() / 7.0, 1e-5, "avg pool")
    # adjoint pairs at full size
    gy = torch.randn(32, 128, 1, m.shape[1], generator=g).to(DEV)
    gx_avg = ops.mapped_avg_unpool(gy, m, 1, x.shape[3], 7, 0)
    _assert_adjoint(yavg, gy, x, gx_avg, 1e-4, "avg pool / unpool")
    gx_max = ops.mapped_max_unpool(gy, idx, m, 1, x.shape[3], 7, 0)
    _assert_adjoint(ymax, gy, x, gx_max, 1e-4, "max pool / unpool")


def test_config4_knn_properties_at_full_size():
    """k = 9 nearest neighbours among the 163 842 level-7 vertices."""
    from mappedconvolutions_b200 import ops
    from mappedconvolutions_b200.util import icosphere as ico
    from mappedconvolutions_b200 import util as mutil
    p = mutil.generate_icosphere(7).get_vertices().t().contiguous().unsqueeze(0).to(DEV)   # (1, 3, N)
    n = p.shape[2]
    idx, dist = ops.knn_forward(p, p, 9)
    idx, dist = idx[0], dist[0]                                             # (9, N)
    assert idx.min().item() >= 1 and idx.max().item() <= n                  # 1-based
    assert torch.equal(idx[0], torch.arange(1, n + 1, device=DEV))          # self match first
    assert (dist[1:] >= dist[:-1]).all()                                    # sorted
    nb = p[0][:, (idx - 1).reshape(-1)].reshape(3, 9, n)
    d2 = ((nb - p[0].unsqueeze(1)) ** 2).sum(0)
    assert torch.allclose(dist * dist, d2, rtol=1e-4, atol=1e-9)             # Euclidean distances
    # brute force on a sample of the queries: same neighbour sets
    q = torch.arange(0, n, 331, device=DEV)
    full = ((p[0][:, q].t().unsqueeze(2) - p[0].unsqueeze(0)) ** 2).sum(1)  # (Q, N)
    want = full.topk(9, dim=1, largest=False).indices + 1
    got = idx[:, q].t()
    assert torch.equal(got.sort(1).values, want.sort(1).values)


def test_config5_encoder_gradients_add_up_over_the_batch():
    """The encoder step of config 5 at full batch: the weight gradients of a batch-64 step equal
    the sum over its two halves (what the batch sharding over ranks relies on)."""
    from mappedconvolutions_b200 import nn as mnn
    from mappedconvolutions_b200.util import icosphere as ico
    torch.manual_seed(5)
    ch, lvl = (3, 64, 128, 256, 256), (7, 6, 5, 5)
    convs = torch.nn.ModuleList(
        [mnn.MappedConvolution(ch[i], ch[i + 1], 7, "nearest") for i in range(4)]).to(DEV).to(torch.bfloat16)
    kmap = {l: ico.vertex_kernel_map(l).to(DEV) for l in (7, 6, 5)}
    pmap = {l: ico.pooling_map(l).to(DEV) for l in (7, 6)}
    pool = mnn.MappedAvgPool(7, "nearest")
    x = _cl(torch.randn(64, 3, 1, ico.num_vertices(7)).to(torch.bfloat16).to(DEV))

    def grads(xin):
        for p in convs.parameters():
            p.grad = None
        h = torch.relu(convs[0](xin, kmap[7]))
        h = pool(h, pmap[7])
        h = torch.relu(convs[1](h, kmap[6]))
        h = pool(h, pmap[6])
        h = torch.relu(convs[2](h, kmap[5]))
        h = torch.relu(convs[3](h, kmap[5]))
        h.float().sum().backward()
        return [p.grad.float().clone() for p in convs.parameters()], h

    whole, out = grads(x)
    assert torch.isfinite(out.float()).all()
    a, _ = grads(_cl(x[:32]))
    b, _ = grads(_cl(x[32:]))
    for gw, ga, gb in zip(whole, a, b):
        H.assert_close(gw, ga + gb, 2e-2, "gradient over the batch")


# Each layer of the config-5 encoder at its REAL size (one batch element, which the oracle finishes
# in seconds): (C_in, C_out, mesh level).  7-tap one-ring maps, nearest, bf16 channels-last.
ENCODER_LAYERS = [(3, 64, 7), (64, 128, 6), (128, 256, 5), (256, 256, 5)]


@pytest.mark.parametrize("cin,cout,level", ENCODER_LAYERS)
def test_config5_layer_against_oracle(cin, cout, level):
    """Forward, input gradient, weight gradient and bias gradient of one encoder layer at its full
    vertex count against the oracle (float32 on the bf16-rounded operands, tolerance 2e-2), and
    element e of a batch-4 call bit-equal to the batch-1 call (no atomics in fwd / dgrad)."""
    from mappedconvolutions_b200 import ops
    from mappedconvolutions_b200.util import icosphere as ico
    g = torch.Generator().manual_seed(50 + level + cin)
    n, K, B = ico.num_vertices(level), 7, 4
    bf = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16)
    x, gy = bf(B, cin, 1, n), bf(B, cout, 1, n)
    w = (torch.randn(cout, cin, K, generator=g) / (cin * K) ** 0.5).to(torch.bfloat16)
    b = bf(cout)
    m = ico.vertex_kernel_map(level)
    xd, gd, md = _cl(x.to(DEV)), _cl(gy.to(DEV)), m.to(DEV)
    y = ops.mapped_conv_forward(xd, md, w.to(DEV), b.to(DEV), K, 0)
    gx, gw, gb = ops.mapped_conv_backward(gd, md, xd, w.to(DEV), b.to(DEV), K, 0)
    e = 2
    y1 = ops.mapped_conv_forward(_cl(xd[e:e + 1]), md, w.to(DEV), b.to(DEV), K, 0)
    g1 = ops.mapped_conv_backward(_cl(gd[e:e + 1]), md, _cl(xd[e:e + 1]), w.to(DEV), b.to(DEV), K, 0)
    assert torch.equal(y1[0], y[e])
    if cin % 64 == 0:   # gather-form input gradient: no atomics, bit for bit
        assert torch.equal(g1[0][0], gx[e])
    else:               # 3-channel first layer: generic input gradient with atomic adds
        H.assert_close(g1[0][0].float(), gx[e].float(), 2e-2, "grad_x batch independence")
    xc, gc = x[e:e + 1].float().contiguous(), gy[e:e + 1].float().contiguous()
    want_y = oracle.mapped_conv_forward(xc, m, w.float(), b.float(), K, 0)
    want_g = oracle.mapped_conv_backward(gc, m, xc, w.float(), b.float(), K, 0)
    H.assert_close(y1.float(), want_y, 2e-2, "y vs oracle")
    H.assert_close(g1[0].float(), want_g[0], 2e-2, "grad_x vs oracle")
    H.assert_close(g1[1].float(), want_g[1], 2e-2, "grad_w vs oracle")
    H.assert_close(g1[2].float(), want_g[2], 2e-2, "grad_b vs oracle")
    # the batch-4 weight gradient is the sum of the per-element ones
    acc = sum(ops.mapped_conv_backward(_cl(gd[i:i + 1]), md, _cl(xd[i:i + 1]), w.to(DEV), b.to(DEV),
                                       K, 0)[1].float() for i in range(B))
    H.assert_close(gw.float(), acc, 2e-2, "grad_w batch sum")


@pytest.mark.parametrize("ch,level", [(64, 7), (128, 6)])
def test_config5_pooling_against_oracle(ch, level):
    """The two average-pooling steps of the encoder (level 7 -> 6 on 64 channels, 6 -> 5 on 128),
    forward and unpooling, bf16 channels-last, one element against the oracle."""
    from mappedconvolutions_b200 import ops
    from mappedconvolutions_b200.util import icosphere as ico
    g = torch.Generator().manual_seed(60 + level)
    n_hi, n_lo = ico.num_vertices(level), ico.num_vertices(level - 1)
    x = torch.randn(2, ch, 1, n_hi, generator=g).to(torch.bfloat16)
    gy = torch.randn(2, ch, 1, n_lo, generator=g).to(torch.bfloat16)
    m = ico.pooling_map(level)
    y = ops.mapped_avg_pool(_cl(x.to(DEV)), m.to(DEV), 7, 0)
    gx = ops.mapped_avg_unpool(_cl(gy.to(DEV)), m.to(DEV), 1, n_hi, 7, 0)
    want_y = oracle.mapped_avg_pool(x[1:2].float().contiguous(), m, 7, 0)
    want_gx = oracle.mapped_avg_unpool(gy[1:2].float().contiguous(), m, 1, n_hi, 7, 0)
    H.assert_close(y[1:2].float(), want_y, 2e-2, "avg pool vs oracle")
    H.assert_close(gx[1:2].float(), want_gx, 2e-2, "avg unpool vs oracle")
