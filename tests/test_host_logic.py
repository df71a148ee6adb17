"""CPU: host-side behaviour of the layer API (argument checks, parameter shapes, the refusal to
run on CPU tensors, the drop-in import names)."""
import math

import pytest
import torch


def test_drop_in_import_names():
    import mapped_convolution.nn as a
    import mapped_convolutions.nn as b
    import mapped_convolution.util as u
    for n in ("MappedConvolution", "MappedTransposedConvolution", "MappedMaxPool", "MappedAvgPool",
              "MappedAvgUnpool", "Resample", "Unresample"):
        assert getattr(a, n) is getattr(b, n)
    assert callable(u.knn)
    import _mapped_convolution_ext._mapped_convolution as m
    assert callable(m.mapped_conv_forward) and callable(m.mapped_conv_backward)
    import _mapped_convolution_ext._knn as k
    assert callable(k.knn_forward)


def test_parameter_shapes_and_init():
    from mapped_convolution.nn import MappedConvolution, MappedTransposedConvolution
    torch.manual_seed(0)
    c = MappedConvolution(6, 10, kernel_size=7, interpolation='nearest')
    assert c.weight.shape == (10, 6, 7) and c.bias.shape == (10,) and c.interp == 0
    s = 1 / math.sqrt(6 * 7)
    assert c.weight.abs().max() <= s and c.bias.abs().max() <= s
    t = MappedTransposedConvolution(6, 10, kernel_size=7, interpolation='bispherical', bias=False)
    assert t.weight.shape == (6, 10, 7) and t.interp == 2
    assert torch.count_nonzero(t.bias) == 0 and t.bias.requires_grad
    assert set(c.state_dict()) == {"weight", "bias"}
    with pytest.raises(AssertionError):
        MappedConvolution(1, 1, 1, interpolation='cubic')


def test_argument_checks_raise_assertion_error():
    from mapped_convolution.nn import MappedConvolution, MappedAvgUnpool, Resample
    layer = MappedConvolution(2, 3, kernel_size=4)
    x = torch.zeros(1, 2, 4, 5)
    m = torch.zeros(4, 5, 4, 2)
    with pytest.raises(AssertionError):
        layer(x[0], m)                       # input not 4-D
    with pytest.raises(AssertionError):
        layer(x, m[..., :1])                 # last map dim != 2
    with pytest.raises(AssertionError):
        layer(x, m.double())                 # dtype mismatch
    with pytest.raises(AssertionError):
        layer(torch.zeros(1, 3, 4, 5), m)    # channel mismatch
    with pytest.raises(AssertionError):
        layer(x, torch.zeros(4, 5, 3, 2))    # kernel size mismatch
    with pytest.raises(AssertionError):
        layer(x, torch.zeros(4, 5, 4, 3, 2), torch.zeros(4, 5, 4, 2))  # P mismatch
    with pytest.raises(AssertionError):
        MappedAvgUnpool(4)(x, 8, 8, torch.zeros(3, 5, 4, 2))           # map grid != input size
    with pytest.raises(AssertionError):
        Resample()(x, torch.zeros(4, 4, 2), (8, 8))


def test_bf16_input_takes_float32_map():
    from mappedconvolutions_b200.nn.checks import check_args
    check_args(torch.zeros(1, 2, 4, 5, dtype=torch.bfloat16), torch.zeros(4, 5, 4, 2), None, 2, 4)
    with pytest.raises(AssertionError):
        check_args(torch.zeros(1, 2, 4, 5, dtype=torch.bfloat16),
                   torch.zeros(4, 5, 4, 2, dtype=torch.bfloat16), None, 2, 4)


def test_cpu_tensors_are_refused_loudly():
    from mapped_convolution.nn import MappedConvolution, Unresample
    from mapped_convolution.util import knn
    with pytest.raises(RuntimeError, match="CUDA only"):
        MappedConvolution(2, 3, kernel_size=4)(torch.zeros(1, 2, 4, 5), torch.zeros(4, 5, 4, 2))
    with pytest.raises(RuntimeError, match="CUDA only"):
        Unresample()(torch.zeros(1, 2, 4, 5), torch.zeros(3, 3, 2))
    with pytest.raises(RuntimeError, match="CUDA only"):
        knn(torch.zeros(1, 3, 8), torch.zeros(1, 3, 8), 2)


def test_product_does_not_import_the_oracle():
    """No module of the product package may reach into oracle/."""
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for pkg in ("mappedconvolutions_b200", "mapped_convolution", "mapped_convolutions",
                "_mapped_convolution_ext"):
        for dp, _, fs in os.walk(os.path.join(root, pkg)):
            for f in fs:
                if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                    src = open(os.path.join(dp, f)).read()
                    assert "oracle" not in src, os.path.join(dp, f)


def test_compiled_extension_carries_the_reference_surface():
    """The PyTorch C++ extension is built in-tree and exports every op function of its ctypes twin."""
    import inspect
    from mappedconvolutions_b200 import build, host, ops
    build.build_torch_ext()
    import importlib
    importlib.reload(host)
    assert host.COMPILED
    public = [n for n, f in inspect.getmembers(ops, inspect.isfunction)
              if not n.startswith("_") and f.__module__ == ops.__name__ and n != "clear_inverse_map_cache"]
    assert len(public) >= 21 and all(hasattr(host.impl, n) for n in public)
    assert host.impl.abi_version() == 2


def _both_bindings():
    from mappedconvolutions_b200 import host, ops
    return [ops] + ([host.impl] if host.COMPILED else [])


@pytest.mark.parametrize("which", [0, 1])
def test_bindings_refuse_mismatched_parameters(which):
    """The C ABI takes raw pointers, so both host bindings check parameter / gradient dtypes and
    shapes before anything reaches it (the reference raises through weight.data<scalar_t>(),
    src/nn/cuda/mapped_convolution_layer.cu:57-65).  The checks come before the device check, so
    they can be exercised with CPU tensors."""
    b = _both_bindings()
    if which >= len(b):
        pytest.skip("compiled extension not built")
    o = b[which]
    x = torch.zeros(2, 4, 5, 6)
    m = torch.zeros(5, 6, 3, 2)
    w, bias = torch.zeros(7, 4, 3), torch.zeros(7)
    gy = torch.zeros(2, 7, 5, 6)
    bf = torch.bfloat16
    # a well-formed CPU call gets as far as the device check
    with pytest.raises(RuntimeError, match="CUDA only"):
        o.mapped_conv_forward(x, m, w, bias, 3, 1)
    with pytest.raises(RuntimeError, match="weight dtype"):
        o.mapped_conv_forward(x.to(bf), m, w, bias, 3, 1)          # fp32 layer fed bf16 input
    with pytest.raises(RuntimeError, match="weight dtype"):
        o.mapped_conv_forward(x.double(), m.double(), w, bias, 3, 1)
    with pytest.raises(RuntimeError, match="bias dtype"):
        o.mapped_conv_forward(x, m, w, bias.double(), 3, 1)
    with pytest.raises(RuntimeError, match="weight must have shape"):
        o.mapped_conv_forward(x, m, torch.zeros(7, 5, 3), bias, 3, 1)  # C_in mismatch
    with pytest.raises(RuntimeError, match="weight must have shape"):
        o.mapped_conv_forward(x, m, torch.zeros(7, 4, 2), bias, 3, 1)  # K mismatch
    with pytest.raises(RuntimeError, match="bias must have"):
        o.mapped_conv_forward(x, m, w, torch.zeros(6), 3, 1)
    with pytest.raises(RuntimeError, match="sample_map.size"):
        o.mapped_conv_forward(x, torch.zeros(5, 6, 4, 2), torch.zeros(7, 4, 4), bias, 3, 1) \
            if False else o.mapped_conv_forward(x, torch.zeros(5, 6, 4, 2), w, bias, 3, 1)
    with pytest.raises(RuntimeError, match="grad_output dtype"):
        o.mapped_conv_backward(gy.double(), m, x, w, bias, 3, 1)
    with pytest.raises(RuntimeError, match="grad_output must have shape"):
        o.mapped_conv_backward(torch.zeros(2, 7, 5, 5), m, x, w, bias, 3, 1)
    # transposed layer: weight (C_in, C_out, K), map of the input's size
    wt = torch.zeros(4, 7, 3)
    with pytest.raises(RuntimeError, match="CUDA only"):
        o.mapped_transposed_conv_forward(x, m, wt, bias, 9, 9, 3, 1)
    with pytest.raises(RuntimeError, match="weight must have shape"):
        o.mapped_transposed_conv_forward(x, m, w, bias, 9, 9, 3, 1)
    with pytest.raises(RuntimeError, match="weight dtype"):
        o.mapped_transposed_conv_backward(torch.zeros(2, 7, 9, 9), m, x, wt.double(), bias, 3, 1)
    with pytest.raises(RuntimeError, match="size of the input"):
        o.mapped_transposed_conv_forward(x, torch.zeros(4, 6, 3, 2), wt, bias, 9, 9, 3, 1)
    # max unpooling: int64 offsets of grad_output's shape
    g = torch.zeros(2, 4, 5, 6)
    with pytest.raises(RuntimeError, match="idx_mask must be int64"):
        o.mapped_max_unpool(g, torch.zeros(2, 4, 5, 6, dtype=torch.int32), m, 8, 8, 3, 0)
    with pytest.raises(RuntimeError, match="idx_mask shape"):
        o.mapped_max_unpool(g, torch.zeros(2, 4, 5, 5, dtype=torch.int64), m, 8, 8, 3, 0)


def test_weighted_maps_fold_only_when_a_tap_fits_one_record():
    """mc_weighted_plan_desc is pure host logic: P points x corners per point (1 nearest, 4 bilinear /
    bispherical) <= 4 folds into the descriptor of a plain bilinear map; everything else is refused."""
    import ctypes
    from mappedconvolutions_b200 import _lib
    L = _lib.lib()
    mk = lambda P, interp, dtype=_lib.MC_BF16: _lib.McDesc(2, 64, 128, 1, 300, 1, 300, 7, P, interp, dtype, _lib.MC_NHWC)
    for P, interp, ok in ((3, 0, True), (4, 0, True), (5, 0, False), (1, 1, True), (1, 2, True), (2, 1, False),
                          (3, 1, False), (0, 0, False)):
        d, f = mk(P, interp), _lib.McDesc()
        rc = L.mc_weighted_plan_desc(ctypes.byref(d), ctypes.byref(f))
        assert (rc == 0) == ok, (P, interp, rc)
        if ok:
            assert (f.P, f.interp, f.C_in, f.C_out, f.K, f.OW) == (0, 1, 64, 128, 7, 300)
            assert L.mc_tapmap_bytes(ctypes.byref(f)) >= 300 * 7 * 32
    d, f = mk(3, 0, _lib.MC_F64), _lib.McDesc()
    assert L.mc_weighted_plan_desc(ctypes.byref(d), ctypes.byref(f)) == -2      # MC_ERR_UNSUPPORTED
    assert L.mc_weighted_plan_desc(ctypes.byref(mk(3, 0)), None) == -1          # MC_ERR_BAD_ARG


def test_utility_entry_points_check_their_arguments_before_touching_the_device():
    from mappedconvolutions_b200 import _lib
    L = _lib.lib()
    assert L.mc_voting_resample_workspace(2, 3, 4, 5, 6) == 2 * 3 * 4 * 5 * 6 * 4
    assert L.mc_voting_resample_workspace(2, 3, 0, 5, 6) == 0
    assert L.mc_cube2rect(_lib.MC_F32, None, 3, 8, 16, 32, 0, None, None) == -1
    assert L.mc_cube2rect(_lib.MC_F32, 16, 3, 8, 16, 32, 2, 16, None) == -1       # unknown interpolation
    assert L.mc_cube2rect(_lib.MC_BF16, 16, 3, 8, 16, 32, 0, 16, None) == -2      # float32 / float64 only
    assert L.mc_voting_resample(None, None, 1, 1, 4, 4, 2, 2, 3, None, 0, None, None) == -1
    assert L.mc_voting_resample(16, 16, 1, 1, 4, 4, 2, 2, 3, None, 0, 16, None) == -3   # MC_ERR_WORKSPACE
    assert L.mc_voting_resample(16, 24, 1, 1, 4, 4, 2, 2, 3, 16, 1 << 20, 16, None) == -1  # map not 16-byte aligned
