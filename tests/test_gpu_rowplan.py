"""Row-plan convolution kernels (maps that are translation invariant along image rows) through the
C ABI, against the oracle (float32 on the bf16-rounded operands, tolerance 2e-2) and against the
general tensor-core kernels of the same library."""
import ctypes

import numpy as np
import pytest
import torch

import helpers as H
from oracle import oracle
from test_rowplan_host import gnomonic_like_map

pytestmark = pytest.mark.gpu


def build_plan(d, m_dev):
    """analysis on the device -> host assembly -> (host plan, device plan) or None"""
    from mappedconvolutions_b200 import _lib
    L = _lib.lib()
    n = L.mc_rowplan_analysis_bytes(d)
    if n == 0:
        return None
    ana = torch.empty(n // 8, dtype=torch.float64, device=m_dev.device)
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(L.mc_rowplan_analyse(d, m_dev.data_ptr(), ana.data_ptr(), st))
    ana_h = np.ascontiguousarray(ana.cpu().numpy())
    if (ana_h.reshape(-1, 3)[:, 2] == 0).any():
        return None
    map_h = np.ascontiguousarray(m_dev.cpu().numpy())
    need = L.mc_rowplan_assemble(d, ana_h.ctypes.data, map_h.ctypes.data, None, 0)
    if need == 0:
        return None
    plan_h = np.zeros(need, dtype=np.int32)
    assert L.mc_rowplan_assemble(d, ana_h.ctypes.data, map_h.ctypes.data, plan_h.ctypes.data, need) == need
    return plan_h, torch.from_numpy(plan_h).to(m_dev.device)


def run(d, direction, src, plan, w, bias, res_shape):
    from mappedconvolutions_b200 import _lib
    L = _lib.lib()
    plan_h, plan_d = plan
    nws = L.mc_conv_rowplan_workspace_bytes(d, plan_h.ctypes.data, direction)
    ws = torch.empty(max(nws, 16), dtype=torch.uint8, device=src.device)
    res = torch.empty(res_shape, dtype=torch.bfloat16, device=src.device).contiguous(
        memory_format=torch.channels_last)
    fn = L.mc_conv_fwd_rowplan if direction == 0 else L.mc_conv_dgrad_rowplan
    _lib.check(fn(d, src.data_ptr(), plan_h.ctypes.data, plan_d.data_ptr(), w.data_ptr(),
                  None if bias is None else bias.data_ptr(), res.data_ptr(), ws.data_ptr(), nws,
                  torch.cuda.current_stream().cuda_stream))
    assert L.mc_device_status(torch.cuda.current_stream().cuda_stream, 1) == 0
    return res


def cl(t):
    return t.contiguous(memory_format=torch.channels_last)


def run_wgrad(d, gy, x, plan):
    from mappedconvolutions_b200 import _lib
    L = _lib.lib()
    plan_h, plan_d = plan
    nws = L.mc_conv_wgrad_rowplan_workspace_bytes(d, plan_h.ctypes.data)
    ws = torch.empty(max(nws, 16), dtype=torch.uint8, device=x.device)
    gw = torch.full((d.C_out, d.C_in, d.K), float("nan"), dtype=torch.float32, device=x.device)
    gb = torch.full((d.C_out,), float("nan"), dtype=torch.float32, device=x.device)
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(L.mc_conv_wgrad_rowplan(d, gy.data_ptr(), x.data_ptr(), plan_h.ctypes.data,
                                       plan_d.data_ptr(), gw.data_ptr(), gb.data_ptr(), ws.data_ptr(),
                                       nws, st))
    assert L.mc_device_status(st, 1) == 0
    return gw, gb


@pytest.mark.parametrize("wrapped,interp,Hh,Ww,B", [(True, 1, 12, 512, 2), (False, 1, 9, 512, 3),
                                                  (True, 2, 7, 1024, 1), (False, 2, 5, 512, 2),
                                                  (True, 1, 3, 512, 19)])  # more images than one MMA pass of the corrections takes
def test_rowplan_forward_and_input_gradient(wrapped, interp, Hh, Ww, B):
    from mappedconvolutions_b200 import _lib
    C, K = 64, 9
    m = gnomonic_like_map(Hh, Ww, wrapped, seed=Hh)
    d = _lib.McDesc(B, C, C, Hh, Ww, Hh, Ww, K, 0, interp, _lib.MC_BF16, _lib.MC_NHWC)
    plan = build_plan(d, m.cuda())
    assert plan is not None
    g = torch.Generator().manual_seed(3)
    bf = torch.bfloat16
    x, gy = torch.randn(B, C, Hh, Ww, generator=g).to(bf), torch.randn(B, C, Hh, Ww, generator=g).to(bf)
    w, b = torch.randn(C, C, K, generator=g).to(bf), torch.randn(C, generator=g).to(bf)
    y = run(d, 0, cl(x.cuda()), plan, w.cuda(), b.cuda(), (B, C, Hh, Ww))
    gx = run(d, 1, cl(gy.cuda()), plan, w.cuda(), None, (B, C, Hh, Ww))
    gw, gb = run_wgrad(d, cl(gy.cuda()), cl(x.cuda()), plan)
    want_y = oracle.mapped_conv_forward(x.float(), m, w.float(), b.float(), K, interp)
    want = oracle.mapped_conv_backward(gy.float(), m, x.float(), w.float(), b.float(), K, interp)
    H.assert_close(y.float(), want_y, 2e-2, "row-plan forward vs oracle")
    H.assert_close(gx.float(), want[0], 2e-2, "row-plan input gradient vs oracle")
    H.assert_close(gw, want[1], 2e-2, "row-plan weight gradient vs oracle")
    H.assert_close(gb, want[2], 2e-2, "row-plan bias gradient vs oracle")


def test_rowplan_on_the_gnomonic_map_matches_the_general_kernels():
    """The benchmark's gnomonic 3 x 3 map (all latitudes, poles included) on a 64 x 512 image."""
    from mappedconvolutions_b200 import _lib, ops
    from mappedconvolutions_b200.util import get_projection_map
    Hh, Ww, C, K, B = 64, 512, 64, 9, 2
    m = get_projection_map((Hh, Ww), (3, 3), "gnomonic").contiguous()
    d = _lib.McDesc(B, C, C, Hh, Ww, Hh, Ww, K, 0, 1, _lib.MC_BF16, _lib.MC_NHWC)
    plan = build_plan(d, m.cuda())
    assert plan is not None
    g = torch.Generator().manual_seed(4)
    bf = torch.bfloat16
    x, gy = torch.randn(B, C, Hh, Ww, generator=g).to(bf), torch.randn(B, C, Hh, Ww, generator=g).to(bf)
    w, b = torch.randn(C, C, K, generator=g).to(bf), torch.randn(C, generator=g).to(bf)
    y = run(d, 0, cl(x.cuda()), plan, w.cuda(), b.cuda(), (B, C, Hh, Ww))
    gx = run(d, 1, cl(gy.cuda()), plan, w.cuda(), None, (B, C, Hh, Ww))
    gw, gb = run_wgrad(d, cl(gy.cuda()), cl(x.cuda()), plan)
    want_y = oracle.mapped_conv_forward(x.float(), m, w.float(), b.float(), K, 1)
    want = oracle.mapped_conv_backward(gy.float(), m, x.float(), w.float(), b.float(), K, 1)
    H.assert_close(y.float(), want_y, 2e-2, "forward vs oracle")
    H.assert_close(gx.float(), want[0], 2e-2, "input gradient vs oracle")
    H.assert_close(gw, want[1], 2e-2, "weight gradient vs oracle")
    H.assert_close(gb, want[2], 2e-2, "bias gradient vs oracle")
    y2 = ops.mapped_conv_forward(cl(x.cuda()), m.cuda(), w.cuda(), b.cuda(), K, 1)
    H.assert_close(y.float(), y2.float(), 2e-2, "forward vs the general kernel")


@pytest.mark.parametrize("dead_row", [None, 3])
def test_rowplan_with_fewer_map_rows_than_image_rows(dead_row):
    """A map grid with half as many rows as the sampled image (vertical stride 2) and taps that leave
    the image at the top and bottom: result rows and source rows differ in count in both directions,
    some source rows are read by no tap of some row pairs, and an odd number of map rows leaves the
    last pair with one row.  dead_row: a map row whose taps all lie outside the image (its result is
    the bias, it has no unit in the weight gradient, and the bias gradient then comes from the
    stand-alone reduction)."""
    from mappedconvolutions_b200 import _lib
    IH, OH, Ww, C, K, B = 14, 7, 512, 64, 9, 2
    g = torch.Generator().manual_seed(5)
    kx = torch.tensor([-1., 0., 1.]).repeat(3).view(1, 1, 9) * 1.5 + 0.3 * torch.rand(OH, 1, 9, generator=g)
    ky = torch.tensor([-1., 0., 1.]).repeat_interleave(3).view(1, 1, 9) * 1.2 + 0.3 * torch.rand(OH, 1, 9, generator=g)
    x_pos = torch.remainder(torch.arange(Ww).view(1, Ww, 1).float() + kx, Ww).expand(OH, Ww, 9)
    y_pos = (2.0 * torch.arange(OH).view(OH, 1, 1).float() + ky).expand(OH, Ww, 9).clone()   # rows -1.5 .. 13.5
    if dead_row is not None:
        y_pos[dead_row] = -10.0
    m = torch.stack((x_pos, y_pos), -1).contiguous()
    d = _lib.McDesc(B, C, C, IH, Ww, OH, Ww, K, 0, 1, _lib.MC_BF16, _lib.MC_NHWC)
    plan = build_plan(d, m.cuda())
    assert plan is not None
    bf = torch.bfloat16
    x, gy = torch.randn(B, C, IH, Ww, generator=g).to(bf), torch.randn(B, C, OH, Ww, generator=g).to(bf)
    w, b = torch.randn(C, C, K, generator=g).to(bf), torch.randn(C, generator=g).to(bf)
    y = run(d, 0, cl(x.cuda()), plan, w.cuda(), b.cuda(), (B, C, OH, Ww))
    gx = run(d, 1, cl(gy.cuda()), plan, w.cuda(), None, (B, C, IH, Ww))
    gw, gb = run_wgrad(d, cl(gy.cuda()), cl(x.cuda()), plan)
    want_y = oracle.mapped_conv_forward(x.float(), m, w.float(), b.float(), K, 1)
    want = oracle.mapped_conv_backward(gy.float(), m, x.float(), w.float(), b.float(), K, 1)
    H.assert_close(y.float(), want_y, 2e-2, "forward vs oracle")
    H.assert_close(gx.float(), want[0], 2e-2, "input gradient vs oracle")
    H.assert_close(gw, want[1], 2e-2, "weight gradient vs oracle")
    H.assert_close(gb, want[2], 2e-2, "bias gradient vs oracle")
