"""Operator surface of the reference's pybind modules, bound to the sm_100a C-ABI library.

Function names, argument order and return values follow the reference's
`_mapped_convolution_ext.<module>` functions (include/nn/layers/*.h, include/util/layers/knn_layer.h
of the reference's package/ext_modules); each docstring cites the one it mirrors.  As in the
reference, outputs are freshly allocated and returned, and inputs must be contiguous and on one
device.  Differences: tensors must be CUDA tensors (there is no CPU path), bf16 activations are
accepted (with a float32 sample map), and a 4-D activation may be channels_last, in which case
the outputs are channels_last too.
"""
import weakref

import torch

from . import _lib
from ._lib import McDesc, check, lib

_DT = {torch.float32: _lib.MC_F32, torch.float64: _lib.MC_F64, torch.bfloat16: _lib.MC_BF16}


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts):
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("mapped convolution ops are CUDA only: got a CPU tensor "
                               "(this build has no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError("all tensors must be on the same device")
    return dev


def _layout(x):
    if x.is_contiguous():
        return _lib.MC_NCHW
    if x.dim() == 4 and x.is_contiguous(memory_format=torch.channels_last):
        return _lib.MC_NHWC
    raise RuntimeError("input must be contiguous")


def _as_layout(t, layout):
    if layout == _lib.MC_NHWC:
        return t.contiguous(memory_format=torch.channels_last)
    return t.contiguous()


def _empty(shape, like, layout, dtype=None):
    fmt = torch.channels_last if layout == _lib.MC_NHWC else torch.contiguous_format
    return torch.empty(shape, dtype=dtype or like.dtype, device=like.device, memory_format=fmt)


def _map_args(x, sample_map, interp_weights):
    """Checks the map / weights tensors; returns (map, weights-or-None)."""
    want = torch.float64 if x.dtype == torch.float64 else torch.float32
    if sample_map.dtype != want:
        if x.dtype == torch.bfloat16 and sample_map.dtype == torch.bfloat16:
            raise RuntimeError("sample map of a bfloat16 input must be float32")
        raise RuntimeError("sample map dtype %s does not match input dtype %s"
                           % (sample_map.dtype, x.dtype))
    if not sample_map.is_contiguous():
        raise RuntimeError("sample_map must be contiguous")
    if interp_weights is not None:
        if interp_weights.dtype != want:
            raise RuntimeError("interp_weights dtype must match the sample map")
        if not interp_weights.is_contiguous():
            raise RuntimeError("interp_weights must be contiguous")
    return sample_map, interp_weights


def _check_conv_args(input, sample_map, weight, bias, w0, w1, n_bias, kernel_size, grad_output=None,
                     grad_shape=None):
    """The C ABI takes raw pointers: parameter / gradient dtypes must equal the input's (the
    reference raises through weight.data<scalar_t>(), src/nn/cuda/mapped_convolution_layer.cu:57-65)
    and the shapes must be the ones the descriptor is built from."""
    if input.dim() != 4:
        raise RuntimeError("input must be 4-D (B, C, H, W)")
    if sample_map.dim() < 4 or sample_map.shape[-1] != 2:
        raise RuntimeError("sample_map must be (OH, OW, K, 2) or (OH, OW, K, P, 2)")
    if weight.dtype != input.dtype:
        raise RuntimeError("weight dtype %s does not match input dtype %s" % (weight.dtype, input.dtype))
    if bias.dtype != input.dtype:
        raise RuntimeError("bias dtype %s does not match input dtype %s" % (bias.dtype, input.dtype))
    if tuple(weight.shape) != (w0, w1, kernel_size):
        raise RuntimeError("weight must have shape (%d, %d, %d), got %s"
                           % (w0, w1, kernel_size, tuple(weight.shape)))
    if bias.numel() != n_bias:
        raise RuntimeError("bias must have %d elements, got %d" % (n_bias, bias.numel()))
    if sample_map.shape[2] != kernel_size:
        raise RuntimeError("sample_map.size(2) = %d does not match kernel_size %d"
                           % (sample_map.shape[2], kernel_size))
    if not weight.is_contiguous() or not bias.is_contiguous():
        raise RuntimeError("weight and bias must be contiguous")
    if grad_output is not None:
        if grad_output.dtype != input.dtype:
            raise RuntimeError("grad_output dtype %s does not match input dtype %s"
                               % (grad_output.dtype, input.dtype))
        if tuple(grad_output.shape) != tuple(grad_shape):
            raise RuntimeError("grad_output must have shape %s, got %s"
                               % (tuple(grad_shape), tuple(grad_output.shape)))


def _desc(x_dtype, layout, B, C_in, C_out, IH, IW, OH, OW, K, P, interp):
    if x_dtype not in _DT:
        raise RuntimeError("unsupported dtype %s (float32, float64, bfloat16)" % x_dtype)
    return McDesc(int(B), int(C_in), int(C_out), int(IH), int(IW), int(OH), int(OW), int(K), int(P),
                  int(interp), _DT[x_dtype], layout)


def _ws(nbytes, device):
    if nbytes == 0:
        return None, 0, None
    t = torch.empty(int(nbytes), dtype=torch.uint8, device=device)
    return t, int(nbytes), t.data_ptr()


def _ptr(t):
    return None if t is None else t.data_ptr()


def _P(interp_weights):
    return 0 if interp_weights is None else int(interp_weights.shape[-1])


# ------------------------------------------------------------------------------------------
# inverse-map cache
# ------------------------------------------------------------------------------------------
# The inverse map depends only on the sample map tensor and the image sizes.  A layer is called
# with the same map tensor step after step, so the last few are kept, keyed by the tensor's
# identity and version counter (an in-place edit of the map invalidates its entry).
_INV_CACHE = []
_INV_CACHE_SIZE = 8


def _cached(kind, d, sample_map, build):
    key = (kind, sample_map.data_ptr(), sample_map._version, tuple(sample_map.shape), d.IH, d.IW,
           d.interp, sample_map.device.index)
    for i, (k, ref, buf) in enumerate(_INV_CACHE):
        if k == key and ref() is sample_map:
            if i:
                _INV_CACHE.insert(0, _INV_CACHE.pop(i))
            return buf
    buf = build()
    _INV_CACHE.insert(0, (key, weakref.ref(sample_map), buf))
    del _INV_CACHE[_INV_CACHE_SIZE:]
    return buf


def _inverse_map(d, sample_map):
    """Inverse map (+ its tap table) of a sample map, built once per map tensor."""
    def build():
        L = lib()
        dev = sample_map.device
        nbytes = L.mc_invmap_bytes(d)
        inv = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        wst, wsn, wsp = _ws(L.mc_invmap_build_workspace_bytes(d), dev)
        check(L.mc_invmap_build(d, sample_map.data_ptr(), inv.data_ptr(), nbytes, wsp, wsn,
                                _stream()))
        return inv
    return _cached("inv", d, sample_map, build)


def _tap_map(d, sample_map):
    """Forward tap table of a sample map (None if the descriptor has no tensor-core path)."""
    L = lib()
    nbytes = L.mc_tapmap_bytes(d)
    if nbytes == 0:
        return None

    def build():
        tab = torch.empty(nbytes, dtype=torch.uint8, device=sample_map.device)
        check(L.mc_tapmap_build(d, sample_map.data_ptr(), tab.data_ptr(), nbytes, _stream()))
        return tab
    return _cached("tap", d, sample_map, build)


def clear_inverse_map_cache():
    del _INV_CACHE[:]


# ------------------------------------------------------------------------------------------
# convolution
# ------------------------------------------------------------------------------------------

def _cl(t):
    return t.contiguous(memory_format=torch.channels_last)


def _a16(t):
    """The tensor-core kernels read rows with 16-byte vector loads: a view that starts off a 16-byte
    boundary (a batch slice, say) is copied into a fresh, aligned allocation."""
    return t if t is None or t.data_ptr() % 16 == 0 else t.clone(memory_format=torch.preserve_format)


def _tensor_core_via_channels_last(input, interp_weights, make_desc):
    """bfloat16 tensors in the reference's NCHW layout: the tensor-core kernels want channels-last,
    and two extra layout passes cost far less than the generic kernels (a factor of ten and more at
    64 channels).  True if the call should be rerouted through channels-last copies."""
    if interp_weights is not None or input.dtype != torch.bfloat16 or input.dim() != 4:
        return False
    if _layout(input) != _lib.MC_NCHW:
        return False
    return lib().mc_conv_fwd_workspace_bytes(make_desc(_lib.MC_NHWC)) > 0


def _conv_forward(input, sample_map, interp_weights, weight, bias, kernel_size, interpolation,
                  _nhwc=False):
    input, sample_map = _a16(input), _a16(sample_map)
    _check_conv_args(input, sample_map, weight, bias, weight.shape[0] if weight.dim() else 0,
                     input.shape[1] if input.dim() > 1 else 0, weight.shape[0] if weight.dim() else 0,
                     kernel_size)
    dev = _need_cuda(input, sample_map, interp_weights, weight, bias)
    if not _nhwc and _tensor_core_via_channels_last(
            input, interp_weights,
            lambda lay: _desc(input.dtype, lay, input.shape[0], input.shape[1], weight.shape[0],
                              input.shape[2], input.shape[3], sample_map.shape[0], sample_map.shape[1],
                              kernel_size, 0, interpolation)):
        return _conv_forward(_cl(input), sample_map, None, weight, bias, kernel_size,
                             interpolation, _nhwc=True).contiguous()
    layout = _lib.MC_NHWC if _nhwc else _layout(input)
    sample_map, interp_weights = _map_args(input, sample_map, interp_weights)
    if not weight.is_contiguous() or not bias.is_contiguous():
        raise RuntimeError("weight and bias must be contiguous")
    B, Cin, IH, IW = input.shape
    Cout = weight.shape[0]
    OH, OW = sample_map.shape[0], sample_map.shape[1]
    d = _desc(input.dtype, layout, B, Cin, Cout, IH, IW, OH, OW, kernel_size, _P(interp_weights),
              interpolation)
    y = _empty((B, Cout, OH, OW), input, layout)
    with torch.cuda.device(dev):
        wst, wsn, wsp = _ws(lib().mc_conv_fwd_workspace_bytes(d), dev)
        tab = _tap_map(d, sample_map) if wsn and interp_weights is None else None
        if tab is not None:  # tensor-core path with the map decoded once per map tensor
            check(lib().mc_conv_fwd_tap(d, input.data_ptr(), tab.data_ptr(), weight.data_ptr(),
                                        bias.data_ptr(), y.data_ptr(), wsp, wsn, _stream()))
        else:
            check(lib().mc_conv_fwd(d, input.data_ptr(), sample_map.data_ptr(),
                                    _ptr(interp_weights), weight.data_ptr(), bias.data_ptr(),
                                    y.data_ptr(), wsp, wsn, _stream()))
    return y


def _contract_first(d):
    """Input gradient as GEMM + gather-sum (mc_conv_dgrad_tapsum) instead of gather-in-the-GEMM: when
    the layer has more output than input channels and the product z fits comfortably."""
    lanes = d.C_in // 8
    # (also square wide layers with a nearest map, where the gather inside the GEMM kernel is slow)
    wider = d.C_out > d.C_in or (d.C_out == d.C_in and d.C_in >= 128 and d.interp not in (1, 2))
    return (d.dtype == _lib.MC_BF16 and d.layout == _lib.MC_NHWC and d.P == 0 and wider
            and d.C_in % 8 == 0 and lanes & (lanes - 1) == 0
            and d.B * d.OH * d.OW * d.K * d.C_in * 2 <= 8 << 30)


def _conv_backward(grad_output, sample_map, interp_weights, input, weight, bias, kernel_size,
                   interpolation, need_input_grad=True, _nhwc=False):
    input, sample_map = _a16(input), _a16(sample_map)
    _check_conv_args(input, sample_map, weight, bias, weight.shape[0] if weight.dim() else 0,
                     input.shape[1] if input.dim() > 1 else 0, weight.shape[0] if weight.dim() else 0,
                     kernel_size, grad_output,
                     (input.shape[0], weight.shape[0], sample_map.shape[0], sample_map.shape[1]))
    dev = _need_cuda(grad_output, sample_map, interp_weights, input, weight, bias)
    if not _nhwc and _tensor_core_via_channels_last(
            input, interp_weights,
            lambda lay: _desc(input.dtype, lay, input.shape[0], input.shape[1], weight.shape[0],
                              input.shape[2], input.shape[3], sample_map.shape[0], sample_map.shape[1],
                              kernel_size, 0, interpolation)):
        g = _conv_backward(_cl(grad_output), sample_map, None, _cl(input), weight, bias, kernel_size,
                           interpolation, need_input_grad, _nhwc=True)
        return [g[0].contiguous() if g[0] is not None else None, g[1], g[2]]
    layout = _lib.MC_NHWC if _nhwc else _layout(input)
    grad_output = _a16(_as_layout(grad_output, layout))
    sample_map, interp_weights = _map_args(input, sample_map, interp_weights)
    B, Cin, IH, IW = input.shape
    Cout = weight.shape[0]
    OH, OW = sample_map.shape[0], sample_map.shape[1]
    d = _desc(input.dtype, layout, B, Cin, Cout, IH, IW, OH, OW, kernel_size, _P(interp_weights),
              interpolation)
    acc = torch.float64 if input.dtype == torch.float64 else torch.float32
    gx = _empty(input.shape, input, layout) if need_input_grad else None
    gw = torch.empty(weight.shape, dtype=acc, device=dev)
    gb = torch.empty((Cout,), dtype=acc, device=dev)
    L = lib()
    with torch.cuda.device(dev):
        inv = _inverse_map(d, sample_map) if need_input_grad and L.mc_conv_dgrad_inv_supported(d) else None
        wst, wsn, wsp = _ws(max(L.mc_conv_dgrad_workspace_bytes(d) if inv is None else
                                L.mc_conv_dgrad_inv_workspace_bytes(d),
                                L.mc_conv_wgrad_workspace_bytes(d)), dev)
        if not need_input_grad:
            pass
        elif inv is not None and _contract_first(d):
            # more output than input channels: contract with the weights first (one dense GEMM), then
            # gather-sum the narrow rows through the inverse map
            g2 = grad_output.permute(0, 2, 3, 1).reshape(B * OH * OW, Cout)   # a view of channels-last
            wr = weight.permute(0, 2, 1).reshape(Cout, kernel_size * Cin)
            z = torch.matmul(g2, wr)
            check(L.mc_conv_dgrad_tapsum(d, z.data_ptr(), inv.data_ptr(), gx.data_ptr(), _stream()))
        elif inv is not None:
            check(L.mc_conv_dgrad_inv(d, grad_output.data_ptr(), inv.data_ptr(), weight.data_ptr(),
                                      None, gx.data_ptr(), wsp, wsn, _stream()))
        else:
            check(L.mc_conv_dgrad(d, grad_output.data_ptr(), sample_map.data_ptr(),
                                  _ptr(interp_weights), weight.data_ptr(), None, gx.data_ptr(), wsp,
                                  wsn, _stream()))
        tab = _tap_map(d, sample_map) if interp_weights is None else None
        rc = -2
        if tab is not None:  # weight / bias gradient on the tensor cores from the prebuilt table
            rc = L.mc_conv_wgrad_tap(d, grad_output.data_ptr(), input.data_ptr(), tab.data_ptr(),
                                     gw.data_ptr(), gb.data_ptr(), _stream())
        if rc != -2:
            check(rc)
        else:  # MC_ERR_UNSUPPORTED: shapes only the generic kernels take
            check(L.mc_conv_wgrad(d, grad_output.data_ptr(), input.data_ptr(),
                                  sample_map.data_ptr(), _ptr(interp_weights), gw.data_ptr(),
                                  gb.data_ptr(), wsp, wsn, _stream()))
    return [gx, gw.to(weight.dtype), gb.to(bias.dtype)]


def mapped_conv_forward(input, sample_map, weight, bias, kernel_size, interpolation):
    """MappedConvForward, include/nn/layers/mapped_convolution_layer.h:64-88."""
    return _conv_forward(input, sample_map, None, weight, bias, kernel_size, interpolation)


def mapped_conv_backward(grad_output, sample_map, input, weight, bias, kernel_size, interpolation,
                         need_input_grad=True, need_weight_grad=True, relu_output=None):
    """MappedConvBackward, include/nn/layers/mapped_convolution_layer.h:90-135.
    Returns [grad_input, grad_weight, grad_bias].  need_input_grad=False (not in the reference's
    signature) skips the input gradient and returns None in its place.  relu_output: the layer's
    output behind a fused ReLU - grad_output is then masked by relu_output > 0 first."""
    if relu_output is not None:
        grad_output = torch.ops.aten.threshold_backward(grad_output, relu_output, 0)
    g = _conv_backward(grad_output, sample_map, None, input, weight, bias, kernel_size,
                       interpolation, need_input_grad)
    return g if need_weight_grad else [g[0], None, None]


def weighted_mapped_conv_forward(input, sample_map, interp_weights, weight, bias, kernel_size,
                                 interpolation):
    """WeightedMappedConvForward, include/nn/layers/weighted_mapped_convolution_layer.h:65-93."""
    return _conv_forward(input, sample_map, interp_weights, weight, bias, kernel_size,
                         interpolation)


def weighted_mapped_conv_backward(grad_output, sample_map, interp_weights, input, weight, bias,
                                  kernel_size, interpolation):
    """WeightedMappedConvBackward, include/nn/layers/weighted_mapped_convolution_layer.h:95-149."""
    return _conv_backward(grad_output, sample_map, interp_weights, input, weight, bias,
                          kernel_size, interpolation)


# ------------------------------------------------------------------------------------------
# transposed convolution
# ------------------------------------------------------------------------------------------

def _tconv_forward(input, sample_map, interp_weights, weight, bias, output_height, output_width,
                   kernel_size, interpolation, _nhwc=False):
    input, sample_map = _a16(input), _a16(sample_map)
    _check_conv_args(input, sample_map, weight, bias, input.shape[1] if input.dim() > 1 else 0,
                     weight.shape[1] if weight.dim() > 1 else 0,
                     weight.shape[1] if weight.dim() > 1 else 0, kernel_size)
    if tuple(sample_map.shape[:2]) != tuple(input.shape[2:]):
        raise RuntimeError("the sample map of a transposed convolution has the size of the input")
    dev = _need_cuda(input, sample_map, interp_weights, weight, bias)
    if not _nhwc and _tensor_core_via_channels_last(
            input, interp_weights,
            lambda lay: _desc(input.dtype, lay, input.shape[0], weight.shape[1], input.shape[1],
                              output_height, output_width, input.shape[2], input.shape[3],
                              kernel_size, 0, interpolation)):
        return _tconv_forward(_cl(input), sample_map, None, weight, bias, output_height, output_width,
                              kernel_size, interpolation, _nhwc=True).contiguous()
    layout = _lib.MC_NHWC if _nhwc else _layout(input)
    sample_map, interp_weights = _map_args(input, sample_map, interp_weights)
    if not weight.is_contiguous() or not bias.is_contiguous():
        raise RuntimeError("weight and bias must be contiguous")
    B, Cin, H, W = input.shape
    Cout = weight.shape[1]
    d = _desc(input.dtype, layout, B, Cin, Cout, output_height, output_width, H, W, kernel_size,
              _P(interp_weights), interpolation)
    y = _empty((B, Cout, int(output_height), int(output_width)), input, layout)
    L = lib()
    # The same layer seen as a convolution: the sampled image carries C_out channels, the map grid
    # C_in.  Its input gradient IS this forward pass, so the gather-form tensor-core dgrad serves.
    ds = _desc(input.dtype, layout, B, Cout, Cin, output_height, output_width, H, W, kernel_size,
               _P(interp_weights), interpolation)
    with torch.cuda.device(dev):
        if interp_weights is None and L.mc_conv_dgrad_inv_supported(ds):
            inv = _inverse_map(ds, sample_map)
            wst, wsn, wsp = _ws(L.mc_conv_dgrad_inv_workspace_bytes(ds), dev)
            check(L.mc_conv_dgrad_inv(ds, input.data_ptr(), inv.data_ptr(), weight.data_ptr(),
                                      bias.data_ptr(), y.data_ptr(), wsp, wsn, _stream()))
            return y
        wst, wsn, wsp = _ws(L.mc_tconv_workspace_bytes(d), dev)
        check(L.mc_tconv_fwd(d, input.data_ptr(), sample_map.data_ptr(), _ptr(interp_weights),
                             weight.data_ptr(), bias.data_ptr(), y.data_ptr(), wsp, wsn, _stream()))
    return y


def _tconv_backward(grad_output, sample_map, interp_weights, input, weight, bias, kernel_size,
                    interpolation, _nhwc=False):
    input, sample_map = _a16(input), _a16(sample_map)
    if grad_output.dim() != 4:
        raise RuntimeError("grad_output must be 4-D")
    _check_conv_args(input, sample_map, weight, bias, input.shape[1] if input.dim() > 1 else 0,
                     weight.shape[1] if weight.dim() > 1 else 0,
                     weight.shape[1] if weight.dim() > 1 else 0, kernel_size, grad_output,
                     (input.shape[0], weight.shape[1], grad_output.shape[2], grad_output.shape[3]))
    if tuple(sample_map.shape[:2]) != tuple(input.shape[2:]):
        raise RuntimeError("the sample map of a transposed convolution has the size of the input")
    dev = _need_cuda(grad_output, sample_map, interp_weights, input, weight, bias)
    if not _nhwc and _tensor_core_via_channels_last(
            input, interp_weights,
            lambda lay: _desc(input.dtype, lay, input.shape[0], weight.shape[1], input.shape[1],
                              grad_output.shape[2], grad_output.shape[3], input.shape[2],
                              input.shape[3], kernel_size, 0, interpolation)):
        g = _tconv_backward(_cl(grad_output), sample_map, None, _cl(input), weight, bias, kernel_size,
                            interpolation, _nhwc=True)
        return [g[0].contiguous(), g[1], g[2]]
    layout = _lib.MC_NHWC if _nhwc else _layout(input)
    grad_output = _a16(_as_layout(grad_output, layout))
    sample_map, interp_weights = _map_args(input, sample_map, interp_weights)
    B, Cin, H, W = input.shape
    Cout = weight.shape[1]
    OHt, OWt = grad_output.shape[2], grad_output.shape[3]
    d = _desc(input.dtype, layout, B, Cin, Cout, OHt, OWt, H, W, kernel_size, _P(interp_weights),
              interpolation)
    acc = torch.float64 if input.dtype == torch.float64 else torch.float32
    gx = _empty(input.shape, input, layout)
    gw = torch.empty(weight.shape, dtype=acc, device=dev)
    gb = torch.empty((Cout,), dtype=acc, device=dev)
    L = lib()
    ds = _desc(input.dtype, layout, B, Cout, Cin, OHt, OWt, H, W, kernel_size, _P(interp_weights),
               interpolation)
    with torch.cuda.device(dev):
        tab = _tap_map(ds, sample_map) if interp_weights is None else None
        if tab is not None and L.mc_conv_fwd_workspace_bytes(ds):
            # tensor-core path: input gradient = forward of the equivalent convolution applied to
            # grad_output; weight gradient = its weight gradient with the two tensors swapped
            wst, wsn, wsp = _ws(L.mc_conv_fwd_workspace_bytes(ds), dev)
            check(L.mc_conv_fwd_tap(ds, grad_output.data_ptr(), tab.data_ptr(), weight.data_ptr(),
                                    None, gx.data_ptr(), wsp, wsn, _stream()))
            rc = L.mc_conv_wgrad_tap(ds, input.data_ptr(), grad_output.data_ptr(), tab.data_ptr(),
                                     gw.data_ptr(), None, _stream())
            if rc == -2:
                rc = L.mc_conv_wgrad(ds, input.data_ptr(), grad_output.data_ptr(),
                                     sample_map.data_ptr(), None, gw.data_ptr(), None, wsp, wsn,
                                     _stream())
            check(rc)
            db = _desc(input.dtype, layout, B, Cout, Cout, OHt, OWt, OHt, OWt, 1, 0, interpolation)
            check(L.mc_bias_grad(db, grad_output.data_ptr(), gb.data_ptr(), _stream()))
            return [gx, gw.to(weight.dtype), gb.to(bias.dtype)]
        wst, wsn, wsp = _ws(L.mc_tconv_workspace_bytes(d), dev)
        check(L.mc_tconv_dgrad(d, grad_output.data_ptr(), sample_map.data_ptr(),
                               _ptr(interp_weights), weight.data_ptr(), gx.data_ptr(), wsp, wsn,
                               _stream()))
        check(L.mc_tconv_wgrad(d, grad_output.data_ptr(), input.data_ptr(), sample_map.data_ptr(),
                               _ptr(interp_weights), gw.data_ptr(), gb.data_ptr(), wsp, wsn,
                               _stream()))
    return [gx, gw.to(weight.dtype), gb.to(bias.dtype)]


def mapped_transposed_conv_forward(input, sample_map, weight, bias, output_height, output_width,
                                   kernel_size, interpolation):
    """MappedTransposedConvForward, include/nn/layers/mapped_transposed_convolution_layer.h:64-92."""
    return _tconv_forward(input, sample_map, None, weight, bias, output_height, output_width,
                          kernel_size, interpolation)


def mapped_transposed_conv_backward(grad_output, sample_map, input, weight, bias, kernel_size,
                                    interpolation):
    """MappedTransposedConvBackward, include/nn/layers/mapped_transposed_convolution_layer.h:94-143."""
    return _tconv_backward(grad_output, sample_map, None, input, weight, bias, kernel_size,
                           interpolation)


def weighted_mapped_transposed_conv_forward(input, sample_map, interp_weights, weight, bias,
                                            output_height, output_width, kernel_size,
                                            interpolation):
    """include/nn/layers/weighted_mapped_transposed_convolution_layer.h:66-98."""
    return _tconv_forward(input, sample_map, interp_weights, weight, bias, output_height,
                          output_width, kernel_size, interpolation)


def weighted_mapped_transposed_conv_backward(grad_output, sample_map, interp_weights, input,
                                             weight, bias, kernel_size, interpolation):
    """include/nn/layers/weighted_mapped_transposed_convolution_layer.h:100-155."""
    return _tconv_backward(grad_output, sample_map, interp_weights, input, weight, bias,
                           kernel_size, interpolation)


# ------------------------------------------------------------------------------------------
# pooling
# ------------------------------------------------------------------------------------------

def _pool_desc(x, sample_map, interp_weights, kernel_size, interpolation, img_hw=None):
    """Descriptor for pooling: x lives on the image for forward, on the map grid for backward."""
    layout = _layout(x)
    B, C = x.shape[0], x.shape[1]
    OH, OW = sample_map.shape[0], sample_map.shape[1]
    IH, IW = (x.shape[2], x.shape[3]) if img_hw is None else img_hw
    return layout, _desc(x.dtype, layout, B, C, C, IH, IW, OH, OW, kernel_size, _P(interp_weights),
                         interpolation)


def _max_pool(input, sample_map, interp_weights, kernel_size, interpolation):
    dev = _need_cuda(input, sample_map, interp_weights)
    sample_map, interp_weights = _map_args(input, sample_map, interp_weights)
    layout, d = _pool_desc(input, sample_map, interp_weights, kernel_size, interpolation)
    shape = (d.B, d.C_in, d.OH, d.OW)
    y = _empty(shape, input, layout)
    idx = _empty(shape, input, layout, dtype=torch.int64)
    with torch.cuda.device(dev):
        check(lib().mc_pool_max_fwd(d, input.data_ptr(), sample_map.data_ptr(),
                                    _ptr(interp_weights), y.data_ptr(), idx.data_ptr(), _stream()))
    return [y, idx]


def _max_unpool(grad_output, idx_mask, sample_map, interp_weights, input_height, input_width,
                kernel_size, interpolation):
    if idx_mask.dtype != torch.int64:
        raise RuntimeError("idx_mask must be int64, got %s" % idx_mask.dtype)
    if tuple(idx_mask.shape) != tuple(grad_output.shape):
        raise RuntimeError("idx_mask shape %s does not match grad_output shape %s"
                           % (tuple(idx_mask.shape), tuple(grad_output.shape)))
    if grad_output.dim() != 4 or tuple(grad_output.shape[2:]) != tuple(sample_map.shape[:2]):
        raise RuntimeError("grad_output must live on the map grid")
    dev = _need_cuda(grad_output, idx_mask, sample_map, interp_weights)
    layout = _layout(idx_mask) if idx_mask.dim() == 4 else _lib.MC_NCHW
    grad_output = _as_layout(grad_output, layout)
    sample_map, interp_weights = _map_args(grad_output, sample_map, interp_weights)
    IH, IW = int(input_height), int(input_width)
    _, d = _pool_desc(grad_output, sample_map, interp_weights, kernel_size, interpolation, (IH, IW))
    gx = _empty((d.B, d.C_in, IH, IW), grad_output, layout)
    L = lib()
    with torch.cuda.device(dev):
        wst, wsn, wsp = _ws(L.mc_scatter_workspace_bytes(d), dev)
        check(L.mc_pool_max_bwd(d, grad_output.data_ptr(), idx_mask.data_ptr(),
                                sample_map.data_ptr(), _ptr(interp_weights), gx.data_ptr(), wsp,
                                wsn, _stream()))
    return gx


def _avg_pool(input, sample_map, interp_weights, kernel_size, interpolation):
    dev = _need_cuda(input, sample_map, interp_weights)
    sample_map, interp_weights = _map_args(input, sample_map, interp_weights)
    layout, d = _pool_desc(input, sample_map, interp_weights, kernel_size, interpolation)
    y = _empty((d.B, d.C_in, d.OH, d.OW), input, layout)
    with torch.cuda.device(dev):
        check(lib().mc_pool_avg_fwd(d, input.data_ptr(), sample_map.data_ptr(),
                                    _ptr(interp_weights), y.data_ptr(), _stream()))
    return y


def _avg_unpool(grad_output, sample_map, interp_weights, input_height, input_width, kernel_size,
                interpolation):
    dev = _need_cuda(grad_output, sample_map, interp_weights)
    layout = _layout(grad_output)
    sample_map, interp_weights = _map_args(grad_output, sample_map, interp_weights)
    IH, IW = int(input_height), int(input_width)
    _, d = _pool_desc(grad_output, sample_map, interp_weights, kernel_size, interpolation, (IH, IW))
    gx = _empty((d.B, d.C_in, IH, IW), grad_output, layout)
    L = lib()
    with torch.cuda.device(dev):
        rc = -2
        if interp_weights is None and L.mc_invmap_bytes(d) > 0:
            # gather through the inverse map (built once per map tensor): no atomics
            inv = _inverse_map(d, sample_map)
            rc = L.mc_pool_avg_bwd_inv(d, grad_output.data_ptr(), inv.data_ptr(), gx.data_ptr(),
                                       _stream())
        if rc != -2:
            check(rc)
        else:
            wst, wsn, wsp = _ws(L.mc_scatter_workspace_bytes(d), dev)
            check(L.mc_pool_avg_bwd(d, grad_output.data_ptr(), sample_map.data_ptr(),
                                    _ptr(interp_weights), gx.data_ptr(), wsp, wsn, _stream()))
    return gx


def mapped_max_pool(input, sample_map, kernel_size, interpolation):
    """MappedMaxPoolForward, include/nn/layers/mapped_max_pooling_layer.h:46-71 -> [out, idx]."""
    return _max_pool(input, sample_map, None, kernel_size, interpolation)


def mapped_max_unpool(grad_output, idx_mask, sample_map, input_height, input_width, kernel_size,
                      interpolation):
    """MappedMaxPoolBackward, include/nn/layers/mapped_max_pooling_layer.h:73-98."""
    return _max_unpool(grad_output, idx_mask, sample_map, None, input_height, input_width,
                       kernel_size, interpolation)


def weighted_mapped_max_pool(input, sample_map, interp_weights, kernel_size, interpolation):
    """include/nn/layers/weighted_mapped_max_pooling_layer.h:42-70."""
    return _max_pool(input, sample_map, interp_weights, kernel_size, interpolation)


def weighted_mapped_max_unpool(grad_output, idx_mask, sample_map, interp_weights, input_height,
                               input_width, kernel_size, interpolation):
    """include/nn/layers/weighted_mapped_max_pooling_layer.h:72-101."""
    return _max_unpool(grad_output, idx_mask, sample_map, interp_weights, input_height,
                       input_width, kernel_size, interpolation)


def mapped_avg_pool(input, sample_map, kernel_size, interpolation):
    """MappedAvgPoolForward, include/nn/layers/mapped_avg_pooling_layer.h:42-64."""
    return _avg_pool(input, sample_map, None, kernel_size, interpolation)


def mapped_avg_unpool(grad_output, sample_map, input_height, input_width, kernel_size,
                      interpolation):
    """MappedAvgPoolBackward, include/nn/layers/mapped_avg_pooling_layer.h:66-88."""
    return _avg_unpool(grad_output, sample_map, None, input_height, input_width, kernel_size,
                       interpolation)


def weighted_mapped_avg_pool(input, sample_map, interp_weights, kernel_size, interpolation):
    """include/nn/layers/weighted_mapped_avg_pooling_layer.h:45-72."""
    return _avg_pool(input, sample_map, interp_weights, kernel_size, interpolation)


def weighted_mapped_avg_unpool(grad_output, sample_map, interp_weights, input_height, input_width,
                               kernel_size, interpolation):
    """include/nn/layers/weighted_mapped_avg_pooling_layer.h:74-107."""
    return _avg_unpool(grad_output, sample_map, interp_weights, input_height, input_width,
                       kernel_size, interpolation)


# ------------------------------------------------------------------------------------------
# resample
# ------------------------------------------------------------------------------------------

def _resample_to_map(input, sample_map, interp_weights, output_height, output_width,
                     interpolation):
    dev = _need_cuda(input, sample_map, interp_weights)
    layout = _layout(input)
    sample_map, interp_weights = _map_args(input, sample_map, interp_weights)
    B, C, H, W = input.shape
    OH, OW = int(output_height), int(output_width)
    d = _desc(input.dtype, layout, B, C, C, OH, OW, H, W, 1, _P(interp_weights), interpolation)
    y = _empty((B, C, OH, OW), input, layout)
    L = lib()
    with torch.cuda.device(dev):
        rc = -2
        if interp_weights is None and L.mc_invmap_bytes(d) > 0:
            inv = _inverse_map(d, sample_map)
            rc = L.mc_resample_scatter_inv(d, input.data_ptr(), inv.data_ptr(), y.data_ptr(),
                                           _stream())
        if rc != -2:
            check(rc)
        else:
            wst, wsn, wsp = _ws(L.mc_scatter_workspace_bytes(d), dev)
            check(L.mc_resample_scatter(d, input.data_ptr(), sample_map.data_ptr(),
                                        _ptr(interp_weights), y.data_ptr(), wsp, wsn, _stream()))
    return y


def _resample_from_map(input, sample_map, interp_weights, interpolation):
    dev = _need_cuda(input, sample_map, interp_weights)
    layout = _layout(input)
    sample_map, interp_weights = _map_args(input, sample_map, interp_weights)
    B, C, H, W = input.shape
    OH, OW = sample_map.shape[0], sample_map.shape[1]
    d = _desc(input.dtype, layout, B, C, C, H, W, OH, OW, 1, _P(interp_weights), interpolation)
    y = _empty((B, C, OH, OW), input, layout)
    with torch.cuda.device(dev):
        check(lib().mc_resample_gather(d, input.data_ptr(), sample_map.data_ptr(),
                                       _ptr(interp_weights), y.data_ptr(), _stream()))
    return y


def resample_to_map(input, sample_map, output_height, output_width, interpolation):
    """ResampleToMap (scatter), include/nn/layers/resample_layer.h:38-60."""
    return _resample_to_map(input, sample_map, None, output_height, output_width, interpolation)


def resample_from_map(input, sample_map, interpolation):
    """ResampleFromMap (gather), include/nn/layers/resample_layer.h:62-80."""
    return _resample_from_map(input, sample_map, None, interpolation)


def weighted_resample_to_map(input, sample_map, interp_weights, output_height, output_width,
                             interpolation):
    """include/nn/layers/weighted_resample_layer.h:49-77."""
    return _resample_to_map(input, sample_map, interp_weights, output_height, output_width,
                            interpolation)


def weighted_resample_from_map(input, sample_map, interp_weights, interpolation):
    """include/nn/layers/weighted_resample_layer.h:79-103."""
    return _resample_from_map(input, sample_map, interp_weights, interpolation)


# ------------------------------------------------------------------------------------------
# knn
# ------------------------------------------------------------------------------------------

def knn_forward(ref, query, k):
    """KNNForward, include/util/layers/knn_layer.h:25-35 -> [idx (B,k,N) int64 1-based, dist]."""
    dev = _need_cuda(ref, query)
    if not ref.is_contiguous() or not query.is_contiguous():
        raise RuntimeError("ref and query must be contiguous")
    if ref.dtype != torch.float32 or query.dtype != torch.float32:
        raise RuntimeError("knn works on float32 points")
    B, D, M = ref.shape
    N = query.shape[2]
    idx = torch.empty((B, k, N), dtype=torch.int64, device=dev)
    dist = torch.empty((B, k, N), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib().mc_knn(ref.data_ptr(), query.data_ptr(), B, D, M, N, int(k), idx.data_ptr(),
                           dist.data_ptr(), _stream()))
    return [idx, dist]


# ------------------------------------------------------------------------------------------
# cube map -> equirectangular image, voting resample
# ------------------------------------------------------------------------------------------

def cube2rect(cubemap, rect_height, rect_width, interpolation):
    """Cube2RectForward, include/util/layers/cube2rect_layer.h:14-45 (src/util/cuda/cube2rect_layer.cu:11-29):
    cubemap (C, D, 6 D) float32 / float64 with faces -z, -x, +z, +x, +y, -y -> (C, rect_height, rect_width)."""
    dev = _need_cuda(cubemap)
    if cubemap.dim() != 3 or cubemap.shape[2] != 6 * cubemap.shape[1]:
        raise RuntimeError("cubemap must be (channels, cube_dim, 6 * cube_dim)")
    if cubemap.dtype not in (torch.float32, torch.float64):
        raise RuntimeError("cube2rect works on float32 / float64 images")
    if interpolation not in (0, 1):
        raise RuntimeError("interpolation must be 0 (nearest) or 1 (bilinear)")
    cubemap = cubemap.contiguous()
    C, D = cubemap.shape[0], cubemap.shape[1]
    rect = torch.empty((C, int(rect_height), int(rect_width)), dtype=cubemap.dtype, device=dev)
    with torch.cuda.device(dev):
        check(lib().mc_cube2rect(_DT[cubemap.dtype], cubemap.data_ptr(), C, D,
                                 int(rect_height), int(rect_width), int(interpolation), rect.data_ptr(), _stream()))
    return rect


def voting_resample_to_map(input, sample_map, output_height, output_width, num_candidates):
    """VotingResampleToMap, include/nn/layers/voting_resample_layer.h:34-58: input (B, C, IH, IW) int64
    labels, sample_map (IH, IW, 2) int64 target (x, y) of every input pixel -> (B, C, OH, OW) int64, the
    label most input pixels brought to each output pixel."""
    dev = _need_cuda(input, sample_map)
    if input.dtype != torch.int64 or sample_map.dtype != torch.int64:
        raise RuntimeError("voting resample works on int64 labels and an int64 map")
    if input.dim() != 4 or tuple(sample_map.shape) != (input.shape[2], input.shape[3], 2):
        raise RuntimeError("input must be (B, C, IH, IW) and sample_map (IH, IW, 2)")
    if num_candidates <= 0:
        raise RuntimeError("num_candidates must be positive")
    input, sample_map = input.contiguous(), sample_map.contiguous()
    B, C, IH, IW = input.shape
    OH, OW, NC = int(output_height), int(output_width), int(num_candidates)
    out = torch.empty((B, C, OH, OW), dtype=torch.int64, device=dev)
    # (vote counters for a slice of the batch at a time: at most ~1 GiB of scratch)
    per_image = lib().mc_voting_resample_workspace(1, C, OH, OW, NC)
    step = max(1, min(B, (1 << 30) // max(1, per_image)))
    ws = torch.empty(per_image * step, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        for b0 in range(0, B, step):
            nb = min(step, B - b0)
            check(lib().mc_voting_resample(input[b0:].data_ptr(), sample_map.data_ptr(), nb, C, IH, IW, OH, OW, NC,
                                           ws.data_ptr(), per_image * nb, out[b0:].data_ptr(), _stream()))
    return out
