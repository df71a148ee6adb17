"""Argument validation of the layer API.

Same conditions and the same failure type (AssertionError) as the reference's
package/layers/nn/layer_utils.py:21-148, with one relaxation: a bfloat16 input takes a float32
sample map (vertex indices beyond 256 are not representable in bfloat16).
"""
from collections.abc import Iterable

import torch

INTERPOLATIONS = {"nearest": 0, "bilinear": 1, "bispherical": 2}


def interp_code(name):
    """'nearest' | 'bilinear' | 'bispherical' -> 0 | 1 | 2
    (package/layers/nn/mapped_convolution_layer.py:81-88)."""
    assert name in INTERPOLATIONS, 'Unsupported interpolation type'
    return INTERPOLATIONS[name]


def _pair(v):
    return v if isinstance(v, Iterable) else (v, v)


def _map_dtype_for(x):
    return torch.float32 if x.dtype == torch.bfloat16 else x.dtype


def check_args(x, sample_map, interp_weights, in_channels, kernel_size):
    """layer_utils.py:125-148.  kernel_size None = a resampling map without the K dimension."""
    has_k = kernel_size is not None
    assert x.dim() == 4, 'Input must have 4 dimensions ({} != 4)'.format(x.dim())
    want = 3 + int(has_k) + int(interp_weights is not None)
    assert sample_map.dim() == want, \
        'Sample map must have {} dimensions ({} != {})'.format(want, sample_map.dim(), want)
    assert sample_map.shape[-1] == 2, \
        'Last dimension of sample map must have size 2 ({} != 2)'.format(sample_map.shape[-1])
    if interp_weights is not None:
        want_w = 3 + int(has_k)
        assert interp_weights.dim() == want_w, \
            'Interpolation weights must have {} dimensions ({} != {})'.format(
                want_w, interp_weights.dim(), want_w)
    md = _map_dtype_for(x)
    assert sample_map.dtype == md, \
        'Input and sample map must be the same dtype ({} != {})'.format(x.dtype, sample_map.dtype)
    if interp_weights is not None:
        assert interp_weights.dtype == md, \
            'Input and interpolation weights must be the same dtype ({} != {})'.format(
                x.dtype, interp_weights.dtype)
    if in_channels is not None:
        assert x.shape[1] == in_channels, \
            'Number of input channels must match weight parameter ({} != {})'.format(
                x.shape[1], in_channels)
    if has_k:
        assert sample_map.shape[2] == kernel_size, \
            'Kernel size of sample map must match weight parameter ({} != {})'.format(
                sample_map.shape[2], kernel_size)
    if interp_weights is not None:
        assert sample_map.shape[-2] == interp_weights.shape[-1], \
            'Sample map and interpolation weights should have the same number of ' \
            'interpolation points ({} != {})'.format(sample_map.shape[-2], interp_weights.shape[-1])


def check_input_map_shape(x, sample_map):
    """layer_utils.py:117-122: the map grid must have the input's spatial size."""
    assert x.shape[2] == sample_map.shape[0] and x.shape[3] == sample_map.shape[1], \
        'Input dimensions 2 and 3 must match sample map dimensions 0 and 1 ' \
        '(({},{}) != ({},{}))'.format(x.shape[2], x.shape[3], sample_map.shape[0],
                                      sample_map.shape[1])
