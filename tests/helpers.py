"""Shared helpers of the parity tests: golden-vector access, the tolerance definition and a
runner that pushes one recorded case through any implementation of the op surface."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_cases(fname):
    """npz with keys '<case>/<field>' -> {case: {field: tensor-or-scalar}}"""
    z = np.load(os.path.join(GOLDEN, fname))
    cases = {}
    for key in z.files:
        case, field = key.rsplit("/", 1)
        v = z[key]
        if v.dtype.kind in "US":
            v = str(v)
        elif v.ndim == 0 and v.dtype.kind in "iub":
            v = int(v)
        else:
            v = torch.from_numpy(v)
        cases.setdefault(case, {})[field] = v
    return cases


def rel_err(new, ref):
    """max |new - ref| / max(|ref|, rms(ref)): the 'relative' error the parity bars are stated
    in.  Element-wise relative error is meaningless next to zero crossings of a long dot product."""
    new, ref = new.detach().double().cpu(), ref.detach().double().cpu()
    assert new.shape == ref.shape, (new.shape, ref.shape)
    if ref.numel() == 0:
        return 0.0
    rms = ref.pow(2).mean().sqrt()
    den = torch.maximum(ref.abs(), rms.expand_as(ref)).clamp_min(1e-300)
    return ((new - ref).abs() / den).max().item()


TOL = {torch.float32: 1e-5, torch.float64: 1e-12, torch.bfloat16: 2e-2}


def assert_close(new, ref, tol, what=""):
    e = rel_err(new, ref)
    assert e <= tol, "%s: relative error %.3e > %.1e" % (what, e, tol)


class Impl:
    """Adapter: an op module + the device its tensors must live on."""

    def __init__(self, ops, device="cpu", layout="nchw"):
        self.ops, self.device, self.layout = ops, device, layout

    def t(self, x):
        if x is None or not isinstance(x, torch.Tensor):
            return x
        x = x.to(self.device)
        if self.layout == "nhwc" and x.dim() == 4 and x.dtype != torch.int64:
            x = x.contiguous(memory_format=torch.channels_last)
        return x

    def act(self, x):
        return self.t(x)

    def plain(self, x):
        """maps / weights / parameters: always plain contiguous"""
        return None if x is None else x.to(self.device).contiguous()


def run_conv(impl, c, transposed=False):
    o = impl.ops
    x, gy = impl.act(c["input"]), impl.act(c["grad_output"])
    w, b, m = impl.plain(c["weight"]), impl.plain(c["bias"]), impl.plain(c["sample_map"])
    iw = impl.plain(c.get("interp_weights"))
    K, interp = c["K"], c["interp"]
    pre = "weighted_" if iw is not None else ""
    name = pre + ("mapped_transposed_conv" if transposed else "mapped_conv")
    fwd, bwd = getattr(o, name + "_forward"), getattr(o, name + "_backward")
    margs = (m, iw) if iw is not None else (m,)
    if transposed:
        y = fwd(x, *margs, w, b, c["oh"], c["ow"], K, interp)
    else:
        y = fwd(x, *margs, w, b, K, interp)
    gx, gw, gb = bwd(gy, *margs, x, w, b, K, interp)
    return dict(output=y, grad_input=gx, grad_weight=gw, grad_bias=gb)


def run_pool(impl, c):
    o = impl.ops
    x, xp, g = impl.act(c["input"]), impl.act(c["input_pos"]), impl.act(c["grad_output"])
    m, iw = impl.plain(c["sample_map"]), impl.plain(c.get("interp_weights"))
    K, interp = c["K"], c["interp"]
    IH, IW = x.shape[2], x.shape[3]
    if iw is not None:
        my, mi = o.weighted_mapped_max_pool(xp, m, iw, K, interp)
        mu = o.weighted_mapped_max_unpool(g, mi, m, iw, IH, IW, K, interp)
        ay = o.weighted_mapped_avg_pool(x, m, iw, K, interp)
        au = o.weighted_mapped_avg_unpool(g, m, iw, IH, IW, K, interp)
    else:
        my, mi = o.mapped_max_pool(xp, m, K, interp)
        mu = o.mapped_max_unpool(g, mi, m, IH, IW, K, interp)
        ay = o.mapped_avg_pool(x, m, K, interp)
        au = o.mapped_avg_unpool(g, m, IH, IW, K, interp)
    return dict(max_output=my, max_idx=mi, max_unpool=mu, avg_output=ay, avg_unpool=au)


def run_resample(impl, c):
    o = impl.ops
    x, xg = impl.act(c["input"]), impl.act(c["grid_input"])
    m, iw = impl.plain(c["sample_map"]), impl.plain(c.get("interp_weights"))
    interp = c["interp"]
    if iw is not None:
        ga = o.weighted_resample_from_map(x, m, iw, interp)
        sc = o.weighted_resample_to_map(xg, m, iw, c["oh"], c["ow"], interp)
    else:
        ga = o.resample_from_map(x, m, interp)
        sc = o.resample_to_map(xg, m, c["oh"], c["ow"], interp)
    return dict(gather_output=ga, scatter_output=sc)


# fields that the reference computes without any reordering freedom: bit-exact on every device
EXACT_FIELDS = {"max_output", "max_idx", "avg_output", "gather_output"}


def compare_case(got, c, tol, what, exact=True):
    for k, v in got.items():
        want = c[k]
        v = v.detach().cpu()
        if v.dtype == torch.int64:
            assert torch.equal(v, want), "%s/%s: index mismatch at %d places" % (
                what, k, (v != want).sum().item())
        elif exact and k in EXACT_FIELDS:
            assert torch.equal(v.contiguous(), want), "%s/%s: not bit-exact (max diff %.3e)" % (
                what, k, (v.double() - want.double()).abs().max().item())
        else:
            assert_close(v, want, tol, "%s/%s" % (what, k))
