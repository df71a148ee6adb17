"""Small tensor helpers of the reference's package/layers/util/util.py."""
import time

import torch


def time_cuda(func, param_list):
    """Runs func(*param_list) between two device synchronisations -> (output, seconds)
    (util.py:6-15)."""
    torch.cuda.synchronize()
    t0 = time.time()
    out = func(*param_list)
    torch.cuda.synchronize()
    return out, time.time() - t0


def _index_view(input, dim, index, batched):
    shape = [1] * input.dim()
    shape[dim] = -1
    if batched:
        shape[0] = input.shape[0]
    want = list(input.shape)
    want[dim] = -1
    return index.view(shape).expand(want)


def batched_index_select(input, dim, index):
    """input (B, ...), index (B, M) or (M,): gathers along `dim` with a per-batch (or shared) index
    list (util.py:18-36)."""
    dim %= input.dim()
    assert index.dim() in (1, 2), "index must have 1 or 2 dimensions ({})".format(index.dim())
    return torch.gather(input, dim, _index_view(input, dim, index, index.dim() == 2))


def batched_scatter(input, dim, index):
    """Scatters input along `dim` to the positions index (M,) of a zero tensor of input's shape
    (util.py:39-50)."""
    dim %= input.dim()
    return torch.zeros_like(input).scatter_(dim, _index_view(input, dim, index, False), input)
