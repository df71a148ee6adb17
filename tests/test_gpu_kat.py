"""GPU: the reference's known-answer tests replayed on the CUDA path (through the C-ABI), plus
the numerical gradient check the reference runs in every test (package/tests/utils.py:92-93)."""
import pytest
import torch
from torch.autograd import gradcheck

import helpers as H
from test_oracle_golden import KAT, check_kat

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", sorted(KAT))
def test_cuda_reproduces_reference_kat(name):
    from mappedconvolutions_b200 import ops
    check_kat(ops, KAT[name], name, dev="cuda", tol=1e-12)


def _layer_for(c):
    import mapped_convolution.nn as nn
    interp = {0: "nearest", 1: "bilinear", 2: "bispherical"}[c["interp"]]
    L = c["layer"]
    if L in ("MappedConvolution", "MappedTransposedConvolution"):
        layer = getattr(nn, L)(c["in_channels"], c["out_channels"], c["kernel_size"], interp).double()
        layer.weight.data = c["weight"].clone()
        layer.bias.data = c["bias"].clone()
        return layer.cuda()
    if L in ("MappedMaxPool", "MappedAvgPool"):
        return getattr(nn, L)(c["kernel_size"], interp)
    return nn.Unresample(interp)


@pytest.mark.parametrize("name", sorted(KAT))
def test_layer_forward_backward_and_gradcheck(name):
    c = KAT[name]
    layer = _layer_for(c)
    x = c["input"].cuda().requires_grad_(True)
    m = c["sample_map"].cuda()
    iw = c["interp_weights"].cuda() if "interp_weights" in c else None
    args = (x, c["oh"], c["ow"], m, iw) if c["layer"] == "MappedTransposedConvolution" else (x, m, iw)
    y = layer(*args)
    assert torch.allclose(y.cpu(), c["expected"], rtol=1e-5, atol=1e-8)
    y.backward(torch.ones_like(y))
    H.assert_close(x.grad, c["grad_input"], 1e-12, name + "/grad_input")
    if "grad_weight" in c:
        H.assert_close(layer.weight.grad, c["grad_weight"], 1e-12, name + "/grad_weight")
        H.assert_close(layer.bias.grad, c["grad_bias"], 1e-12, name + "/grad_bias")
    assert gradcheck(layer, args)
