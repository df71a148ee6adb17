"""Python face of the plain-C oracle (oracle/mc_oracle.c).  TEST INFRASTRUCTURE ONLY.

Functions take and return CPU torch tensors (float32 / float64, NCHW contiguous) and carry the
names and argument orders of the reference's pybind functions, so a test can swap this module,
oracle.ref.ops() and the CUDA ops freely.  bfloat16 inputs are upcast to float32 by the caller.
"""
import ctypes
import os
import subprocess

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmc_oracle.so")
_lib = None


def build():
    subprocess.run(["make", "-C", HERE, "libmc_oracle.so"], check=True, capture_output=True)
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        _lib = ctypes.CDLL(LIB_PATH)
    return _lib


def _suf(t):
    assert t.dtype in (torch.float32, torch.float64) and not t.is_cuda
    return "_f32" if t.dtype == torch.float32 else "_f64"


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _c(*ts):
    return [None if t is None else t.contiguous() for t in ts]


def _call(name, like, *args):
    fn = getattr(lib(), name + _suf(like))
    fn.restype = None
    conv = []
    for a in args:
        if a is None or isinstance(a, torch.Tensor):
            conv.append(_p(a))
        else:
            conv.append(ctypes.c_int(int(a)))
    fn(*conv)


def _P(iw):
    return 0 if iw is None else iw.shape[-1]


# ---- conv ---------------------------------------------------------------------------------
def weighted_mapped_conv_forward(input, sample_map, interp_weights, weight, bias, K, interp):
    input, sample_map, interp_weights, weight, bias = _c(input, sample_map, interp_weights, weight, bias)
    B, Cin, IH, IW = input.shape
    Cout, OH, OW = weight.shape[0], sample_map.shape[0], sample_map.shape[1]
    y = torch.empty(B, Cout, OH, OW, dtype=input.dtype)
    _call("oracle_conv_fwd", input, input, sample_map, interp_weights, weight, bias, y, B, Cin, Cout,
          IH, IW, OH, OW, K, _P(interp_weights), interp)
    return y


def mapped_conv_forward(input, sample_map, weight, bias, K, interp):
    return weighted_mapped_conv_forward(input, sample_map, None, weight, bias, K, interp)


def weighted_mapped_conv_backward(grad_output, sample_map, interp_weights, input, weight, bias, K,
                                  interp):
    grad_output, sample_map, interp_weights, input, weight = _c(grad_output, sample_map,
                                                                interp_weights, input, weight)
    B, Cin, IH, IW = input.shape
    Cout, OH, OW = weight.shape[0], sample_map.shape[0], sample_map.shape[1]
    gx = torch.empty_like(input)
    gw = torch.empty_like(weight)
    gb = torch.empty(Cout, dtype=input.dtype)
    dims = (B, Cin, Cout, IH, IW, OH, OW, K, _P(interp_weights), interp)
    _call("oracle_conv_dgrad", input, grad_output, sample_map, interp_weights, weight, gx, *dims)
    _call("oracle_conv_wgrad", input, grad_output, input, sample_map, interp_weights, gw, gb, *dims)
    return [gx, gw, gb]


def mapped_conv_backward(grad_output, sample_map, input, weight, bias, K, interp):
    return weighted_mapped_conv_backward(grad_output, sample_map, None, input, weight, bias, K, interp)


# ---- transposed conv ------------------------------------------------------------------------
def weighted_mapped_transposed_conv_forward(input, sample_map, interp_weights, weight, bias, oh, ow,
                                            K, interp):
    input, sample_map, interp_weights, weight, bias = _c(input, sample_map, interp_weights, weight, bias)
    B, Cin, H, W = input.shape
    Cout = weight.shape[1]
    y = torch.empty(B, Cout, int(oh), int(ow), dtype=input.dtype)
    _call("oracle_tconv_fwd", input, input, sample_map, interp_weights, weight, bias, y, B, Cin, Cout,
          H, W, oh, ow, K, _P(interp_weights), interp)
    return y


def mapped_transposed_conv_forward(input, sample_map, weight, bias, oh, ow, K, interp):
    return weighted_mapped_transposed_conv_forward(input, sample_map, None, weight, bias, oh, ow, K,
                                                   interp)


def weighted_mapped_transposed_conv_backward(grad_output, sample_map, interp_weights, input, weight,
                                             bias, K, interp):
    grad_output, sample_map, interp_weights, input, weight = _c(grad_output, sample_map,
                                                                interp_weights, input, weight)
    B, Cin, H, W = input.shape
    Cout, OH, OW = weight.shape[1], grad_output.shape[2], grad_output.shape[3]
    gx = torch.empty_like(input)
    gw = torch.empty_like(weight)
    gb = torch.empty(Cout, dtype=input.dtype)
    dims = (B, Cin, Cout, H, W, OH, OW, K, _P(interp_weights), interp)
    _call("oracle_tconv_dgrad", input, grad_output, sample_map, interp_weights, weight, gx, *dims)
    _call("oracle_tconv_wgrad", input, grad_output, input, sample_map, interp_weights, gw, gb, *dims)
    return [gx, gw, gb]


def mapped_transposed_conv_backward(grad_output, sample_map, input, weight, bias, K, interp):
    return weighted_mapped_transposed_conv_backward(grad_output, sample_map, None, input, weight,
                                                    bias, K, interp)


# ---- pooling --------------------------------------------------------------------------------
def weighted_mapped_max_pool(input, sample_map, interp_weights, K, interp, cuda_init=True):
    """cuda_init=True: start value -FLT_MAX (the reference's CUDA build, the semantics the product
    implements); False: numeric_limits<T>::min() (the reference's CPU build)."""
    input, sample_map, interp_weights = _c(input, sample_map, interp_weights)
    B, C, IH, IW = input.shape
    OH, OW = sample_map.shape[0], sample_map.shape[1]
    y = torch.empty(B, C, OH, OW, dtype=input.dtype)
    idx = torch.empty(B, C, OH, OW, dtype=torch.int64)
    _call("oracle_max_pool", input, input, sample_map, interp_weights, y, idx, B, C, IH, IW, OH, OW,
          K, _P(interp_weights), interp, int(cuda_init))
    return [y, idx]


def mapped_max_pool(input, sample_map, K, interp, cuda_init=True):
    return weighted_mapped_max_pool(input, sample_map, None, K, interp, cuda_init)


def weighted_mapped_max_unpool(grad_output, idx_mask, sample_map, interp_weights, IH, IW, K, interp):
    grad_output, idx_mask, sample_map, interp_weights = _c(grad_output, idx_mask, sample_map,
                                                          interp_weights)
    B, C, OH, OW = grad_output.shape
    gx = torch.empty(B, C, int(IH), int(IW), dtype=grad_output.dtype)
    _call("oracle_max_unpool", grad_output, grad_output, idx_mask, sample_map, interp_weights, gx, B,
          C, IH, IW, OH, OW, K, _P(interp_weights), interp)
    return gx


def mapped_max_unpool(grad_output, idx_mask, sample_map, IH, IW, K, interp):
    return weighted_mapped_max_unpool(grad_output, idx_mask, sample_map, None, IH, IW, K, interp)


def weighted_mapped_avg_pool(input, sample_map, interp_weights, K, interp):
    input, sample_map, interp_weights = _c(input, sample_map, interp_weights)
    B, C, IH, IW = input.shape
    OH, OW = sample_map.shape[0], sample_map.shape[1]
    y = torch.empty(B, C, OH, OW, dtype=input.dtype)
    _call("oracle_avg_pool", input, input, sample_map, interp_weights, y, B, C, IH, IW, OH, OW, K,
          _P(interp_weights), interp)
    return y


def mapped_avg_pool(input, sample_map, K, interp):
    return weighted_mapped_avg_pool(input, sample_map, None, K, interp)


def weighted_mapped_avg_unpool(grad_output, sample_map, interp_weights, IH, IW, K, interp):
    grad_output, sample_map, interp_weights = _c(grad_output, sample_map, interp_weights)
    B, C, OH, OW = grad_output.shape
    gx = torch.empty(B, C, int(IH), int(IW), dtype=grad_output.dtype)
    _call("oracle_avg_unpool", grad_output, grad_output, sample_map, interp_weights, gx, B, C, IH, IW,
          OH, OW, K, _P(interp_weights), interp)
    return gx


def mapped_avg_unpool(grad_output, sample_map, IH, IW, K, interp):
    return weighted_mapped_avg_unpool(grad_output, sample_map, None, IH, IW, K, interp)


# ---- resample -------------------------------------------------------------------------------
def weighted_resample_from_map(input, sample_map, interp_weights, interp):
    input, sample_map, interp_weights = _c(input, sample_map, interp_weights)
    B, C, IH, IW = input.shape
    OH, OW = sample_map.shape[0], sample_map.shape[1]
    y = torch.empty(B, C, OH, OW, dtype=input.dtype)
    _call("oracle_resample_gather", input, input, sample_map, interp_weights, y, B, C, IH, IW, OH, OW,
          _P(interp_weights), interp)
    return y


def resample_from_map(input, sample_map, interp):
    return weighted_resample_from_map(input, sample_map, None, interp)


def weighted_resample_to_map(input, sample_map, interp_weights, OH, OW, interp):
    """input lives on the map grid; (OH, OW) is the image written into."""
    input, sample_map, interp_weights = _c(input, sample_map, interp_weights)
    B, C, H, W = input.shape
    y = torch.empty(B, C, int(OH), int(OW), dtype=input.dtype)
    _call("oracle_resample_scatter", input, input, sample_map, interp_weights, y, B, C, OH, OW, H, W,
          _P(interp_weights), interp)
    return y


def resample_to_map(input, sample_map, OH, OW, interp):
    return weighted_resample_to_map(input, sample_map, None, OH, OW, interp)


# ---- knn ------------------------------------------------------------------------------------
def knn_forward(ref, query, k):
    ref, query = ref.contiguous().float(), query.contiguous().float()
    B, D, M = ref.shape
    N = query.shape[2]
    idx = torch.empty(B, k, N, dtype=torch.int64)
    dist = torch.empty(B, k, N, dtype=torch.float32)
    fn = lib().oracle_knn
    fn.restype = None
    fn(_p(ref), _p(query), *(ctypes.c_int(int(v)) for v in (B, D, M, N, k)), _p(idx), _p(dist))
    return [idx, dist]


# ---- voting resample, cube2rect -----------------------------------------------------------------
def voting_resample_to_map(input, sample_map, OH, OW, num_candidates):
    input, sample_map = input.contiguous(), sample_map.contiguous()
    assert input.dtype == torch.int64 and sample_map.dtype == torch.int64
    B, C, IH, IW = input.shape
    out = torch.empty(B, C, OH, OW, dtype=torch.int64)
    fn = lib().oracle_voting_resample
    fn.restype = None
    fn(_p(input), _p(sample_map), *(ctypes.c_int(int(v)) for v in (B, C, IH, IW, OH, OW, num_candidates)),
       _p(out))
    return out


def cube2rect(cubemap, rect_height, rect_width, interp):
    cubemap = cubemap.contiguous()
    C, D = cubemap.shape[0], cubemap.shape[1]
    rect = torch.empty(C, rect_height, rect_width, dtype=cubemap.dtype)
    _call("oracle_cube2rect", cubemap, cubemap, C, D, rect_height, rect_width, interp, rect)
    return rect
