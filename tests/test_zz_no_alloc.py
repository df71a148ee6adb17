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


def test_static_scratch_call_leaves_device_memory_untouched():
    """What the entry point is for: no device memory is obtained or released by the call.  After a
    first call (which looks the array's address up) the free memory of the device and the caching
    allocator's reservation are the same before and after further calls, and two calls queued back
    to back on one stream with different weights both give their own result."""
    from mappedconvolutions_b200 import _lib
    lib = _lib.lib()
    x, w1, b1, m, full = _case(5, 2, 64, 16, 32, 16, 32, 9, 1)
    _, w2, b2, _, _ = _case(6, 2, 64, 16, 32, 16, 32, 9, 1)
    d = _lib.McDesc(*full, _lib.MC_BF16, _lib.MC_NHWC)
    st = torch.cuda.current_stream().cuda_stream
    mk = lambda: torch.empty((2, 64, 16, 32), dtype=torch.bfloat16, device="cuda",
                             memory_format=torch.channels_last)
    y1, y2, r1, r2 = mk(), mk(), mk(), mk()
    n = lib.mc_conv_fwd_workspace_bytes(d)
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    for w, b, r in ((w1, b1, r1), (w2, b2, r2)):
        _lib.check(lib.mc_conv_fwd(d, x.data_ptr(), m.data_ptr(), None, w.data_ptr(), b.data_ptr(),
                                   r.data_ptr(), ws.data_ptr(), n, st))
    _lib.check(lib.mc_conv_fwd_static_scratch(d, x.data_ptr(), m.data_ptr(), w1.data_ptr(),
                                              b1.data_ptr(), y1.data_ptr(), st))   # set-up call
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    reserved0 = torch.cuda.memory_reserved()
    for _ in range(3):
        _lib.check(lib.mc_conv_fwd_static_scratch(d, x.data_ptr(), m.data_ptr(), w1.data_ptr(),
                                                  b1.data_ptr(), y1.data_ptr(), st))
        _lib.check(lib.mc_conv_fwd_static_scratch(d, x.data_ptr(), m.data_ptr(), w2.data_ptr(),
                                                  b2.data_ptr(), y2.data_ptr(), st))
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0 and torch.cuda.memory_reserved() == reserved0
    assert torch.equal(y1, r1) and torch.equal(y2, r2) and not torch.equal(y1, y2)
