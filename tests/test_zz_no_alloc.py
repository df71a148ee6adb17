"""GPU: the forward entry point that brings its own scratch memory.

mc_conv_fwd_static_scratch() exists for callers that may not allocate device memory at call time
(a plugin running inside another framework's step, a server whose memory was partitioned at
start-up): the weight re-layout buffer that mc_conv_fwd() takes from the caller lives in a fixed
array inside the library instead.  It must give exactly the result of mc_conv_fwd(), call after
call, although every call reuses the same array.  This file sorts last so that a run that stops at
the first failure has already executed every other test.
"""
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu


def _case(seed, B, Cin, IH, IW, OH, OW, K, interp):
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    x = torch.randn(B, Cin, IH, IW, generator=g).to(bf).cuda().contiguous(
        memory_format=torch.channels_last)
    w = torch.randn(64, Cin, K, generator=g).to(bf).cuda()
    b = torch.randn(64, generator=g).to(bf).cuda()
    m = (torch.rand(OH, OW, K, 2, generator=g) * torch.tensor([IW + 1.0, IH + 1.0]) - 1.0).cuda()
    return x, w, b, m.contiguous(), (B, Cin, 64, IH, IW, OH, OW, K, 0, interp)


def _both(lib, _lib, x, w, b, m, dims):
    d = _lib.McDesc(*dims, _lib.MC_BF16, _lib.MC_NHWC)
    st = torch.cuda.current_stream().cuda_stream
    shape = (dims[0], 64, dims[5], dims[6])
    y_ref = torch.empty(shape, dtype=torch.bfloat16, device="cuda", memory_format=torch.channels_last)
    y_new = torch.full_like(y_ref, float("nan"))
    n = lib.mc_conv_fwd_workspace_bytes(d)
    assert n > 0, "expected the tensor-core path for this shape"
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    _lib.check(lib.mc_conv_fwd(d, x.data_ptr(), m.data_ptr(), None, w.data_ptr(), b.data_ptr(),
                               y_ref.data_ptr(), ws.data_ptr(), n, st))
    _lib.check(lib.mc_conv_fwd_static_scratch(d, x.data_ptr(), m.data_ptr(), w.data_ptr(),
                                              b.data_ptr(), y_new.data_ptr(), st))
    torch.cuda.synchronize()
    assert lib.mc_device_status(st, 1) == 0
    return y_ref, y_new


def test_static_scratch_forward_matches_the_regular_entry_point_twice():
    from mappedconvolutions_b200 import _lib
    lib = _lib.lib()
    # two calls in a row that use different amounts of the shared array, different weights and
    # different interpolation modes: nothing of the first call may leak into the second
    for seed, dims in ((1, (2, 64, 16, 32, 16, 32, 9, 1)), (2, (1, 128, 9, 20, 8, 16, 4, 0))):
        x, w, b, m, full = _case(seed, *dims)
        y_ref, y_new = _both(lib, _lib, x, w, b, m, full)
        H.assert_close(y_new.float(), y_ref.float(), 2e-2, "static-scratch forward")
        assert torch.equal(y_new, y_ref)  # same kernel, same operands: bit-identical


def test_static_scratch_rejects_what_does_not_fit():
    from mappedconvolutions_b200 import _lib
    lib = _lib.lib()
    limit = lib.mc_conv_fwd_static_scratch_limit()
    x, w, b, m, full = _case(3, 1, 128, 8, 16, 8, 16, 6, 1)      # 6 * 128 * 64 * 2 = 98 304 bytes
    assert 6 * 128 * 64 * 2 > limit
    d = _lib.McDesc(*full, _lib.MC_BF16, _lib.MC_NHWC)
    y = torch.empty((1, 64, 8, 16), dtype=torch.bfloat16, device="cuda",
                    memory_format=torch.channels_last)
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.mc_conv_fwd_static_scratch(d, x.data_ptr(), m.data_ptr(), w.data_ptr(), b.data_ptr(),
                                        y.data_ptr(), st)
    assert rc == -6 and b"limit" in lib.mc_strerror(rc)
    # and a shape the tensor-core forward does not take at all is refused, not silently rerouted
    d2 = _lib.McDesc(1, 64, 40, 8, 16, 8, 16, 3, 0, 1, _lib.MC_BF16, _lib.MC_NHWC)  # C_out % 64 != 0
    assert lib.mc_conv_fwd_static_scratch(d2, x.data_ptr(), m.data_ptr(), w.data_ptr(),
                                          b.data_ptr(), y.data_ptr(), st) == -2
