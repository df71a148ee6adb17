"""autograd.Function wrappers: each op's backward is another op of the same library.

Pairing follows the reference's package/layers/nn/*.py: conv fwd <-> (dgrad, wgrad, dbias);
max pool <-> max unpool through the stored tap offsets; avg pool <-> avg unpool;
Resample (scatter) <-> Unresample (gather).
"""
import torch
from torch.autograd import Function

from ..host import COMPILED as FUSED_RELU  # the compiled extension takes relu=True
from ..host import impl as ops


class MappedConvFn(Function):
    """package/layers/nn/mapped_convolution_layer.py:15-59"""

    @staticmethod
    def forward(ctx, x, weight, bias, sample_map, kernel_size, interp, interp_weights=None,
                relu=False):
        ctx.k, ctx.interp, ctx.relu = int(kernel_size), int(interp), bool(relu)
        if interp_weights is not None:
            y = ops.weighted_mapped_conv_forward(x, sample_map, interp_weights, weight, bias,
                                                 ctx.k, ctx.interp)
            if relu:
                y = torch.relu_(y)
        elif relu and FUSED_RELU:
            # the activation runs in the convolution's epilogue: no separate pass over y
            y = ops.mapped_conv_forward(x, sample_map, weight, bias, ctx.k, ctx.interp, relu=True)
        else:
            y = ops.mapped_conv_forward(x, sample_map, weight, bias, ctx.k, ctx.interp)
            if relu:
                y = torch.relu_(y)
        ctx.save_for_backward(x, weight, bias, sample_map, interp_weights, y if relu else None)
        return y

    @staticmethod
    def backward(ctx, gy):
        x, weight, bias, sample_map, iw, y = ctx.saved_tensors
        # gradient of the activation, from its own output: y > 0 <=> pre-activation > 0
        if iw is not None:
            if ctx.relu:
                gy = torch.ops.aten.threshold_backward(gy, y, 0)  # one pass: gy where y > 0, else 0
            gx, gw, gb = ops.weighted_mapped_conv_backward(gy, sample_map, iw, x, weight, bias,
                                                           ctx.k, ctx.interp)
        else:
            # (the op masks grad_output itself - inside the weight-gradient kernel where it can)
            gx, gw, gb = ops.mapped_conv_backward(gy, sample_map, x, weight, bias, ctx.k,
                                                  ctx.interp, need_input_grad=ctx.needs_input_grad[0],
                                                  relu_output=y if ctx.relu else None)
        return gx, gw, gb, None, None, None, None, None


class MappedTransposedConvFn(Function):
    """package/layers/nn/mapped_transposed_convolution_layer.py:15-61"""

    @staticmethod
    def forward(ctx, x, weight, bias, sample_map, oh, ow, kernel_size, interp,
                interp_weights=None):
        ctx.save_for_backward(x, weight, bias, sample_map, interp_weights)
        ctx.k, ctx.interp = int(kernel_size), int(interp)
        if interp_weights is not None:
            return ops.weighted_mapped_transposed_conv_forward(
                x, sample_map, interp_weights, weight, bias, oh, ow, ctx.k, ctx.interp)
        return ops.mapped_transposed_conv_forward(x, sample_map, weight, bias, oh, ow, ctx.k,
                                                  ctx.interp)

    @staticmethod
    def backward(ctx, gy):
        x, weight, bias, sample_map, iw = ctx.saved_tensors
        if iw is not None:
            gx, gw, gb = ops.weighted_mapped_transposed_conv_backward(
                gy, sample_map, iw, x, weight, bias, ctx.k, ctx.interp)
        else:
            gx, gw, gb = ops.mapped_transposed_conv_backward(gy, sample_map, x, weight, bias,
                                                             ctx.k, ctx.interp)
        return gx, gw, gb, None, None, None, None, None, None


class MappedMaxPoolFn(Function):
    """package/layers/nn/mapped_max_pooling_layer.py:12-55"""

    @staticmethod
    def forward(ctx, x, sample_map, kernel_size, interp, interp_weights=None):
        k, interp = int(kernel_size), int(interp)
        if interp_weights is not None:
            y, idx = ops.weighted_mapped_max_pool(x, sample_map, interp_weights, k, interp)
        else:
            y, idx = ops.mapped_max_pool(x, sample_map, k, interp)
        ctx.mark_non_differentiable(idx)
        ctx.save_for_backward(idx, sample_map, interp_weights)
        ctx.k, ctx.interp, ctx.hw = k, interp, (x.shape[2], x.shape[3])
        return y, idx

    @staticmethod
    def backward(ctx, gy, _gidx=None):
        idx, sample_map, iw = ctx.saved_tensors
        if iw is not None:
            gx = ops.weighted_mapped_max_unpool(gy, idx, sample_map, iw, ctx.hw[0], ctx.hw[1],
                                                ctx.k, ctx.interp)
        else:
            gx = ops.mapped_max_unpool(gy, idx, sample_map, ctx.hw[0], ctx.hw[1], ctx.k,
                                       ctx.interp)
        return gx, None, None, None, None


class MappedAvgPoolFn(Function):
    """package/layers/nn/mapped_avg_pooling_layer.py:12-53"""

    @staticmethod
    def forward(ctx, x, sample_map, kernel_size, interp, interp_weights=None):
        ctx.k, ctx.interp, ctx.hw = int(kernel_size), int(interp), (x.shape[2], x.shape[3])
        ctx.save_for_backward(sample_map, interp_weights)
        if interp_weights is not None:
            return ops.weighted_mapped_avg_pool(x, sample_map, interp_weights, ctx.k, ctx.interp)
        return ops.mapped_avg_pool(x, sample_map, ctx.k, ctx.interp)

    @staticmethod
    def backward(ctx, gy):
        sample_map, iw = ctx.saved_tensors
        if iw is not None:
            gx = ops.weighted_mapped_avg_unpool(gy, sample_map, iw, ctx.hw[0], ctx.hw[1], ctx.k,
                                                ctx.interp)
        else:
            gx = ops.mapped_avg_unpool(gy, sample_map, ctx.hw[0], ctx.hw[1], ctx.k, ctx.interp)
        return gx, None, None, None, None


class MappedAvgUnpoolFn(Function):
    """package/layers/nn/mapped_avg_pooling_layer.py:80-121.  The reference passes the weighted
    arguments in an order its own extension does not accept (:93-94); the evident intent,
    (x, map, weights, oh, ow, k, interp), is what runs here."""

    @staticmethod
    def forward(ctx, x, oh, ow, sample_map, kernel_size, interp, interp_weights=None):
        ctx.k, ctx.interp = int(kernel_size), int(interp)
        ctx.save_for_backward(sample_map, interp_weights)
        if interp_weights is not None:
            return ops.weighted_mapped_avg_unpool(x, sample_map, interp_weights, oh, ow, ctx.k,
                                                  ctx.interp)
        return ops.mapped_avg_unpool(x, sample_map, oh, ow, ctx.k, ctx.interp)

    @staticmethod
    def backward(ctx, gy):
        sample_map, iw = ctx.saved_tensors
        if iw is not None:
            gx = ops.weighted_mapped_avg_pool(gy, sample_map, iw, ctx.k, ctx.interp)
        else:
            gx = ops.mapped_avg_pool(gy, sample_map, ctx.k, ctx.interp)
        return gx, None, None, None, None, None, None


class ResampleFn(Function):
    """Scatter input samples to mapped locations; package/layers/nn/resample_layer.py:14-48"""

    @staticmethod
    def forward(ctx, x, sample_map, output_shape, interp, interp_weights=None):
        ctx.interp = int(interp)
        ctx.save_for_backward(sample_map, interp_weights)
        oh, ow = int(output_shape[0]), int(output_shape[1])
        if interp_weights is not None:
            return ops.weighted_resample_to_map(x, sample_map, interp_weights, oh, ow, ctx.interp)
        return ops.resample_to_map(x, sample_map, oh, ow, ctx.interp)

    @staticmethod
    def backward(ctx, gy):
        sample_map, iw = ctx.saved_tensors
        if iw is not None:
            gx = ops.weighted_resample_from_map(gy, sample_map, iw, ctx.interp)
        else:
            gx = ops.resample_from_map(gy, sample_map, ctx.interp)
        return gx, None, None, None, None


class UnresampleFn(Function):
    """Gather at mapped locations; package/layers/nn/resample_layer.py:82-110"""

    @staticmethod
    def forward(ctx, x, sample_map, interp, interp_weights=None):
        ctx.interp, ctx.hw = int(interp), (x.shape[2], x.shape[3])
        ctx.save_for_backward(sample_map, interp_weights)
        if interp_weights is not None:
            return ops.weighted_resample_from_map(x, sample_map, interp_weights, ctx.interp)
        return ops.resample_from_map(x, sample_map, ctx.interp)

    @staticmethod
    def backward(ctx, gy):
        sample_map, iw = ctx.saved_tensors
        if iw is not None:
            gx = ops.weighted_resample_to_map(gy, sample_map, iw, ctx.hw[0], ctx.hw[1], ctx.interp)
        else:
            gx = ops.resample_to_map(gy, sample_map, ctx.hw[0], ctx.hw[1], ctx.interp)
        return gx, None, None, None
