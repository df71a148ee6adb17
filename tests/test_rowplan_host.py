"""Row plans (sample maps that are translation invariant along image rows): the host-side planner
mc_rowplan_assemble, checked without a GPU.  The plan is evaluated in float64 with plain torch - what
the kernels compute: shifted windows times effective weights, then the fix-up of the missing
right-hand corner of column W - 1 - and compared with the oracle's mapped convolution."""
import ctypes

import numpy as np
import pytest
import torch

from mappedconvolutions_b200 import _lib
from oracle import oracle

TOL = 1e-3


def analyse(m, IW):
    """What rowinv_analyse_kernel computes, in numpy: (OH, K, 3) of cx, cy, kind."""
    m = m.double().numpy()
    OH, OW, K, _ = m.shape
    px, py = m[..., 0], m[..., 1]
    x = np.arange(OW)[None, :, None]
    ref = px[:, OW // 2, :] - OW // 2
    d = px - x - ref[:, None, :]
    dw = np.fmod(d + IW * 0.5, IW)
    dw = np.where(dw < 0, dw + IW, dw) - IW * 0.5
    bad_plain = ~(np.abs(d) <= TOL).all(1)
    bad_wrap = ~((np.abs(dw) <= TOL) & (px >= 0) & (px < IW)).all(1)
    bad_y = ~(np.abs(py - py[:, OW // 2:OW // 2 + 1, :]) <= TOL).all(1)
    kind = np.where(bad_y, 0, (~bad_plain).astype(int) | (2 * (~bad_wrap & (OW == IW)).astype(int)))
    return np.ascontiguousarray(np.stack([ref + dw.mean(1), py.mean(1), kind.astype(np.float64)], -1))


def assemble(d, ana, m):
    L = _lib.lib()
    mh = np.ascontiguousarray(m.float().numpy())
    n = L.mc_rowplan_assemble(d, ana.ctypes.data, mh.ctypes.data, None, 0)
    if n == 0:
        return None
    plan = np.zeros(n, dtype=np.int32)
    assert L.mc_rowplan_assemble(d, ana.ctypes.data, mh.ctypes.data, plan.ctypes.data, n) == n
    return plan


HDR = 8   # magic, total, OH, OW, IH, IW, K, interp
DIR = 18  # ints per direction block


def direction(plan, i):
    f = plan[HDR + DIR * i: HDR + DIR * (i + 1)]
    names = ("rows nwin nslot ncon nskip ngroup max_win max_slot off_row off_win off_slot off_coff "
             "off_ctap off_cw off_skip off_group nwgunit off_wgunit").split()
    return dict(zip(names, (int(v) for v in f)))


def evaluate(plan, i, src, weight, res_hw, transpose, pairs=False):
    """float64 evaluation of direction i of the plan.  src (B, C, SH, SW).  pairs: the windows and
    slots come from the plan for pairs of result rows (directions 2, 3: a slot has one contribution
    list per row of the pair), the corrections from the per-row plan as always."""
    D = direction(plan, i + 2 if pairs else i)
    B, C, SH, SW = src.shape
    RH, RW = res_hw
    Wt = weight.double()
    out = torch.zeros(B, Wt.shape[1] if transpose else Wt.shape[0], RH, RW, dtype=torch.float64)
    row_off = plan[D["off_row"]: D["off_row"] + D["rows"] + 1]
    win = plan[D["off_win"]: D["off_win"] + 4 * D["nwin"]].reshape(-1, 4)
    shift = plan[D["off_slot"]: D["off_slot"] + D["nslot"]]
    coff = plan[D["off_coff"]: D["off_coff"] + D["nslot"] + 1]
    ctap = plan[D["off_ctap"]: D["off_ctap"] + D["ncon"]]
    cw = plan[D["off_cw"]: D["off_cw"] + D["ncon"]].view(np.float32)
    xs = torch.arange(RW)
    s64 = src.double()
    if pairs:
        coff = plan[D["off_coff"]: D["off_coff"] + 2 * D["nslot"] + 1]
        assert D["rows"] == (RH + 1) // 2
    for r in range(D["rows"]):
        for w in range(row_off[r], row_off[r + 1]):
            srow, dx0, first, packed = (int(v) for v in win[w])
            nsl, span, mode = packed & 0xFF, (packed >> 8) & 0xFF, packed >> 16
            assert span <= 32 and nsl >= 1
            for s in range(first, first + nsl):
                sx = xs + dx0 + int(shift[s])
                if mode == 1:
                    ok, sx = torch.ones(RW, dtype=torch.bool), torch.remainder(sx, SW)
                else:
                    ok, sx = (sx >= 0) & (sx < SW), sx.clamp(0, SW - 1)
                for sub in range(2 if pairs else 1):
                    v, row = (2 * s + sub, 2 * r + sub) if pairs else (s, r)
                    if coff[v] == coff[v + 1]:
                        continue
                    assert row < RH
                    E = sum(float(cw[c]) * Wt[:, :, int(ctap[c])] for c in range(coff[v], coff[v + 1]))
                    if transpose:
                        E = E.t()
                    out[:, :, row, :] += torch.einsum("oc,bcn->bon", E, s64[:, :, srow, :][:, :, sx] * ok)
    D = direction(plan, i)
    skip = plan[D["off_skip"]: D["off_skip"] + 6 * D["nskip"]].reshape(-1, 6)
    for row, col, srow, scol, k, wb in skip:
        w = float(np.array([wb], dtype=np.int32).view(np.float32)[0])
        Wk = Wt[:, :, int(k)].t() if transpose else Wt[:, :, int(k)]
        out[:, :, row, col] += w * torch.einsum("oc,bc->bo", Wk, s64[:, :, srow, scol])
    return out


def gnomonic_like_map(H, W, wrapped, seed=0):
    """Row-invariant 3 x 3 kernel map: per-row horizontal spread and fractional positions."""
    g = torch.Generator().manual_seed(seed)
    spread = 1.0 + 3.0 * torch.rand(H, 1, 1, generator=g)
    kx = torch.tensor([-1., 0., 1.]).repeat(3).view(1, 1, 9) * spread + 0.3 * torch.rand(H, 1, 9, generator=g)
    ky = torch.tensor([-1., 0., 1.]).repeat_interleave(3).view(1, 1, 9) * 1.1 + 0.3 * torch.rand(H, 1, 9, generator=g)
    x = torch.arange(W).view(1, W, 1).float() + kx
    y = torch.arange(H).view(H, 1, 1).float() + ky.expand(H, W, 9)
    if wrapped:
        x = torch.remainder(x, W)
    return torch.stack((x.expand(H, W, 9), y), -1).contiguous()


@pytest.mark.parametrize("wrapped,interp,H", [(True, 1, 6), (False, 1, 5), (True, 2, 7), (False, 2, 6)])
def test_plan_reproduces_the_mapped_convolution(wrapped, interp, H):
    W, C, K, B = 512, 64, 9, 2
    m = gnomonic_like_map(H, W, wrapped)
    d = _lib.McDesc(B, C, C, H, W, H, W, K, 0, interp, _lib.MC_BF16, _lib.MC_NHWC)
    plan = assemble(d, analyse(m, W), m)
    assert plan is not None, "a row-invariant map was refused"
    g = torch.Generator().manual_seed(1)
    x, gy = torch.randn(B, C, H, W, generator=g), torch.randn(B, C, H, W, generator=g)
    w, b = torch.randn(C, C, K, generator=g) * 0.1, torch.zeros(C)
    want_y = oracle.mapped_conv_forward(x, m, w, b, K, interp)
    want_gx = oracle.mapped_conv_backward(gy, m, x, w, b, K, interp)[0]
    got_y = evaluate(plan, 0, x, w, (H, W), False)
    got_gx = evaluate(plan, 1, gy, w, (H, W), True)
    # the plan uses ONE position per (row, tap); the map's float32 positions wobble by ~1e-4 px
    assert (got_y - want_y).abs().max().item() <= 2e-3 * want_y.abs().max().item()
    assert (got_gx - want_gx).abs().max().item() <= 2e-3 * want_gx.abs().max().item()
    # the same through the plan for pairs of rows (what the forward / input-gradient kernels run on)
    pair_y = evaluate(plan, 0, x, w, (H, W), False, pairs=True)
    pair_gx = evaluate(plan, 1, gy, w, (H, W), True, pairs=True)
    assert (pair_y - got_y).abs().max().item() <= 1e-9 * want_y.abs().max().item()
    assert (pair_gx - got_gx).abs().max().item() <= 1e-9 * want_gx.abs().max().item()
    # corrections exist exactly where the seam matters: bilinear on wrapped positions
    nskip = direction(plan, 0)["nskip"]
    assert (nskip > 0) == (wrapped and interp == 1)


def test_the_benchmark_map_has_a_plan_and_others_do_not():
    from mappedconvolutions_b200.util import get_projection_map
    H, W, K = 64, 512, 9
    d = _lib.McDesc(1, 64, 64, H, W, H, W, K, 0, 1, _lib.MC_BF16, _lib.MC_NHWC)
    m = get_projection_map((H, W), (3, 3), "gnomonic").contiguous()
    plan = assemble(d, analyse(m, W), m)
    assert plan is not None
    D = direction(plan, 0)
    assert D["rows"] == H and D["max_win"] <= 64 and D["max_slot"] <= 128 and D["nskip"] > 0
    # weight-gradient units: every window of every row exactly once, at most 8 slot pairs each,
    # largest unit first
    wg = plan[D["off_wgunit"]: D["off_wgunit"] + 4 * D["nwgunit"]].reshape(-1, 4)
    win = plan[D["off_win"]: D["off_win"] + 4 * D["nwin"]].reshape(-1, 4)
    row_off = plan[D["off_row"]: D["off_row"] + D["rows"] + 1]
    by_start = wg[np.argsort(wg[:, 1], kind="stable")]
    assert wg[:, 2].sum() == D["nwin"] and by_start[0, 1] == 0
    assert (by_start[1:, 1] == by_start[:-1, 1] + by_start[:-1, 2]).all()
    pairs = []
    for r, w0, nw, s0 in wg:
        assert row_off[r] <= w0 and w0 + nw <= row_off[r + 1] and s0 == win[w0, 2]
        pairs.append(int(sum(((win[w0:w0 + nw, 3] & 0xFF) + 1) // 2)))
    assert max(pairs) <= 8 and pairs == sorted(pairs, reverse=True)
    # a jittered map is not row invariant; neither is a map whose rows move vertically
    g = torch.Generator().manual_seed(2)
    mj = m + 0.01 * torch.rand(m.shape, generator=g)
    assert assemble(d, analyse(mj, W), mj) is None
    m2 = m.clone()
    m2[:, ::2, :, 1] += 0.5
    assert assemble(d, analyse(m2, W), m2) is None
    # shapes without row-plan kernels
    d2 = _lib.McDesc(1, 32, 64, H, W, H, W, K, 0, 1, _lib.MC_BF16, _lib.MC_NHWC)
    assert _lib.lib().mc_rowplan_analysis_bytes(d2) == 0 and assemble(d2, analyse(m, W), m) is None
