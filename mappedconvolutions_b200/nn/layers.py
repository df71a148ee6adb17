"""nn.Module layer API, constructor and forward signatures as in the reference's
package/layers/nn/__init__.py:6-10."""
import math

import torch
import torch.nn as nn

from . import functions as F
from .checks import check_args, check_input_map_shape, interp_code


class _ConvBase(nn.Module):
    """Parameters and initialisation shared by the two convolution layers:
    weight U(-s, s), bias U(-s, s) with s = 1/sqrt(in_channels * kernel_size); bias=False keeps a
    zero, still trainable, bias parameter (package/layers/nn/mapped_convolution_layer.py:90-108)."""

    def __init__(self, in_channels, out_channels, kernel_size, interpolation, bias, transposed):
        super().__init__()
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = kernel_size
        self.interp = interp_code(interpolation)
        wshape = (in_channels, out_channels, kernel_size) if transposed else \
            (out_channels, in_channels, kernel_size)
        self.weight = nn.Parameter(torch.empty(*wshape))
        self.bias = nn.Parameter(torch.empty(out_channels))
        self.reset_parameters()
        if not bias:
            self.bias = nn.Parameter(torch.zeros(out_channels))

    def reset_parameters(self):
        s = 1.0 / math.sqrt(self.in_channels * self.kernel_size)
        with torch.no_grad():
            self.weight.uniform_(-s, s)
            self.bias.uniform_(-s, s)


class MappedConvolution(_ConvBase):
    """out[b, :, p] = W . [interp(x[b], sample_map[p, k]) for every channel and tap k] + bias.

    forward(x (B,C,IH,IW), sample_map (OH,OW,K,2) of (x, y) locations,
            interp_weights=None | (OH,OW,K,P) with sample_map (OH,OW,K,P,2)) -> (B,Cout,OH,OW)
    package/layers/nn/mapped_convolution_layer.py:62-121
    """

    def __init__(self, in_channels, out_channels, kernel_size=1, interpolation='bilinear',
                 bias=True, *, activation=None):
        """activation (keyword only, not in the reference): None, or 'relu' to get
        max(0, conv(x) + bias) from the convolution kernel itself instead of a separate
        element-wise pass; the layer then stands for conv followed by nn.ReLU."""
        super().__init__(in_channels, out_channels, kernel_size, interpolation, bias, False)
        assert activation in (None, 'relu'), 'activation must be None or "relu"'
        self.activation = activation

    def forward(self, x, sample_map, interp_weights=None):
        check_args(x, sample_map, interp_weights, self.in_channels, self.kernel_size)
        return F.MappedConvFn.apply(x, self.weight, self.bias, sample_map, self.kernel_size,
                                    self.interp, interp_weights, self.activation == 'relu')


class MappedTransposedConvolution(_ConvBase):
    """The map has the input's size and points into the (oh, ow) output.

    forward(x (B,C,IH,IW), oh, ow, sample_map (IH,IW,K,2), interp_weights=None) -> (B,Cout,oh,ow)
    package/layers/nn/mapped_transposed_convolution_layer.py:64-121
    """

    def __init__(self, in_channels, out_channels, kernel_size=1, interpolation='bilinear',
                 bias=True):
        super().__init__(in_channels, out_channels, kernel_size, interpolation, bias, True)

    def forward(self, x, oh, ow, sample_map, interp_weights=None):
        check_args(x, sample_map, interp_weights, self.in_channels, self.kernel_size)
        check_input_map_shape(x, sample_map)
        return F.MappedTransposedConvFn.apply(x, self.weight, self.bias, sample_map, oh, ow,
                                              self.kernel_size, self.interp, interp_weights)


class _PoolBase(nn.Module):
    def __init__(self, kernel_size, interpolation):
        super().__init__()
        self.kernel_size = kernel_size
        self.interp = interp_code(interpolation)


class MappedMaxPool(_PoolBase):
    """package/layers/nn/mapped_max_pooling_layer.py:58-90"""

    def __init__(self, kernel_size, interpolation='bilinear', return_indices=False):
        super().__init__(kernel_size, interpolation)
        self.return_indices = return_indices

    def forward(self, x, sample_map, interp_weights=None):
        check_args(x, sample_map, interp_weights, None, self.kernel_size)
        y, idx = F.MappedMaxPoolFn.apply(x, sample_map, self.kernel_size, self.interp,
                                         interp_weights)
        return (y, idx) if self.return_indices else y


class MappedAvgPool(_PoolBase):
    """package/layers/nn/mapped_avg_pooling_layer.py:56-77"""

    def __init__(self, kernel_size, interpolation='bilinear'):
        super().__init__(kernel_size, interpolation)

    def forward(self, x, sample_map, interp_weights=None):
        check_args(x, sample_map, interp_weights, None, self.kernel_size)
        return F.MappedAvgPoolFn.apply(x, sample_map, self.kernel_size, self.interp,
                                       interp_weights)


class MappedAvgUnpool(_PoolBase):
    """package/layers/nn/mapped_avg_pooling_layer.py:124-154"""

    def __init__(self, kernel_size, interpolation='bilinear'):
        super().__init__(kernel_size, interpolation)

    def forward(self, x, oh, ow, sample_map, interp_weights=None):
        check_args(x, sample_map, interp_weights, None, self.kernel_size)
        check_input_map_shape(x, sample_map)
        return F.MappedAvgUnpoolFn.apply(x, oh, ow, sample_map, self.kernel_size, self.interp,
                                         interp_weights)


class Resample(nn.Module):
    """Scatter: every input element is added at its mapped real-valued output location.
    forward(x, sample_map (IH,IW,2), output_shape (OH,OW), interp_weights=None)
    package/layers/nn/resample_layer.py:51-79"""

    def __init__(self, interpolation='bilinear'):
        super().__init__()
        self.interp = interp_code(interpolation)

    def forward(self, x, sample_map, output_shape, interp_weights=None):
        check_args(x, sample_map, interp_weights, None, None)
        check_input_map_shape(x, sample_map)
        return F.ResampleFn.apply(x, sample_map, output_shape, self.interp, interp_weights)


class Unresample(nn.Module):
    """Gather: a mapped convolution with unit weight, no bias and one tap.
    forward(x, sample_map (OH,OW,2), interp_weights=None)
    package/layers/nn/resample_layer.py:113-140"""

    def __init__(self, interpolation='bilinear'):
        super().__init__()
        self.interp = interp_code(interpolation)

    def forward(self, x, sample_map, interp_weights=None):
        check_args(x, sample_map, interp_weights, None, None)
        return F.UnresampleFn.apply(x, sample_map, self.interp, interp_weights)


def _pair(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v)


class _GridConvBase(nn.Module):
    """The reference's two ordinary grid convolutions - its own im2col + GEMM code, kept there as
    a yardstick for the mapped layers (package/layers/nn/convolution_layer.py:34-75,
    transposed_convolution_layer.py:33-74).  Here they are the same modules (constructor,
    parameter shapes, initialisation, output sizes) on top of torch's convolutions: a grid
    convolution is not part of the mapped-convolution path and the library convolution is the
    right tool for it.

    Initialisation as in the reference: the weight is drawn once per kernel dimension (the last
    draw, U(-s, s) with s = 1/sqrt(in_channels * kh * kw), stays), then the bias with the same s,
    so that a seeded construction yields the reference's parameters."""

    def __init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation, transposed):
        super().__init__()
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = _pair(kernel_size)
        self.padding = _pair(padding)
        self.stride = _pair(stride)
        self.dilation = _pair(dilation)
        first = (in_channels, out_channels) if transposed else (out_channels, in_channels)
        self.weight = nn.Parameter(torch.empty(*first, *self.kernel_size))
        self.bias = nn.Parameter(torch.empty(out_channels))
        self.reset_parameters()

    def reset_parameters(self):
        n = self.in_channels
        with torch.no_grad():
            for k in self.kernel_size:
                n *= k
                s = 1.0 / math.sqrt(n)
                self.weight.uniform_(-s, s)
            self.bias.uniform_(-s, s)


class Convolution(_GridConvBase):
    """forward(x (B, C_in, H, W)) -> (B, C_out, (H + 2 p - d (k - 1) - 1) / s + 1, ...), the output size of
    src/nn/cpp/convolution_layer.cpp:17-24.  package/layers/nn/convolution_layer.py:34-75"""

    def __init__(self, in_channels, out_channels, kernel_size=1, stride=1, padding=0, dilation=1):
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, False)

    def forward(self, x):
        return torch.nn.functional.conv2d(x, self.weight, self.bias, self.stride, self.padding, self.dilation)


class TransposedConvolution(_GridConvBase):
    """forward(x (B, C_in, H, W)) -> (B, C_out, s (H - 1) + d (k - 1) + 1 - 2 p, ...), the output size of
    src/nn/cpp/transposed_convolution_layer.cpp:54-57; weight (C_in, C_out, kh, kw).
    package/layers/nn/transposed_convolution_layer.py:33-74"""

    def __init__(self, in_channels, out_channels, kernel_size=1, stride=1, padding=0, dilation=1):
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, True)

    def forward(self, x):
        return torch.nn.functional.conv_transpose2d(x, self.weight, self.bias, self.stride, self.padding, 0, 1,
                                                    self.dilation)
