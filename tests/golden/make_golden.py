"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own CPU code.

Needs the reference checkout ($MC_REFERENCE_ROOT, or a directory `reference` beside this repository) and its CPU extensions built by
oracle/build_ref.py.  It is run by hand when the fixtures need refreshing; the tests only read
the .npz files it writes, never the reference.

Three files are produced:

  kat.npz           every CPU known-answer test of the reference's package/tests/ is executed
                    unchanged, with hooks that record the layer set-up, the inputs, the output of
                    the reference's CPU extension, the gradients of its backward pass and the
                    literal expected tensor the test asserts against.
  random_small.npz  seeded random cases for every op of the hot path (all interpolation modes,
                    weighted and unweighted maps, out-of-range samples, float32 and float64),
                    outputs computed with the reference's CPU extension.
  config1.npz       the float32 3->16 channel, 64x128, K=9 jittered-grid case, forward + backward.
"""
import argparse
import importlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.dont_write_bytecode = True

from oracle import ref  # noqa: E402


def _np(t):
    return t.detach().cpu().numpy()


# ------------------------------------------------------------------------------------------------
# Part A: the reference's own known-answer tests, instrumented
# ------------------------------------------------------------------------------------------------
def capture_kats(ref_root):
    pkg = os.path.join(ROOT, "oracle", "_ref", "pkg")
    os.makedirs(pkg, exist_ok=True)
    link = os.path.join(pkg, "mapped_convolution")
    if not os.path.islink(link):
        os.symlink(os.path.join(ref_root, "package", "layers"), link)
    sys.path[:0] = [os.path.join(ROOT, "oracle", "_ref"), pkg,
                    os.path.join(ref_root, "package", "tests")]

    import torch.testing as tt
    cur = {}
    out = {}

    def assert_allclose(actual, expected, *a, **k):
        # torch >= 2 no longer broadcasts (B,C,H,W) against (H,W); the reference's tests rely on it
        e = expected.expand_as(actual)
        assert torch.allclose(actual, e, rtol=1e-5, atol=1e-8), "reference KAT failed"
        cur["expected"] = e.clone()

    tt.assert_allclose = assert_allclose
    utils = importlib.import_module("utils")

    def wrap(name, has_ohow):
        orig = getattr(utils, name)

        def hooked(layer, *args, **kw):
            res = orig(layer, *args, **kw)
            cur["layer"] = type(layer).__name__
            cur["interp"] = int(layer.interp)
            for attr in ("kernel_size", "in_channels", "out_channels"):
                if hasattr(layer, attr):
                    cur[attr] = int(getattr(layer, attr))
            if hasattr(layer, "weight"):
                cur["weight"] = layer.weight.data.clone()
                cur["bias"] = layer.bias.data.clone()
                cur["grad_weight"] = layer.weight.grad.clone()
                cur["grad_bias"] = layer.bias.grad.clone()
            x = kw["input"]
            cur["input"] = x.detach().clone()
            cur["grad_input"] = x.grad.clone()
            cur["sample_map"] = kw["sample_map"].clone()
            if kw.get("interp_weights") is not None:
                cur["interp_weights"] = kw["interp_weights"].clone()
            if has_ohow:
                cur["oh"], cur["ow"] = int(kw["oh"]), int(kw["ow"])
            cur["output"] = res[0].detach().clone()
            cur["gradcheck"] = bool(res[3])
            return res

        setattr(utils, name, hooked)

    wrap("mapped_conv_test", False)
    wrap("mapped_transposed_conv_test", True)
    wrap("mapped_pool_test", False)
    wrap("mapped_resample_test", False)

    n = 0
    for modname in ("test_mapped_convolution", "test_mapped_transposed_convolution",
                    "test_mapped_pooling", "test_resample"):
        mod = importlib.import_module(modname)
        for fname in sorted(dir(mod)):
            if not (fname.startswith("test_") and fname.endswith("_cpu")):
                continue
            cur.clear()
            getattr(mod, fname)()  # raises if the reference fails its own test
            assert cur["gradcheck"], fname
            case = "%s::%s" % (modname, fname)
            for k, v in cur.items():
                out["%s/%s" % (case, k)] = _np(v) if isinstance(v, torch.Tensor) else np.asarray(v)
            n += 1
            print("KAT ok:", case)
    return out, n


# ------------------------------------------------------------------------------------------------
# Part B: seeded random cases through the reference's pybind functions
# ------------------------------------------------------------------------------------------------
def random_cases():
    R = ref.ops()
    out = {}
    g = torch.Generator().manual_seed(1234)

    def rnd(*s, dt):
        return torch.randn(*s, generator=g, dtype=dt)

    def uni(*s, dt):
        return torch.rand(*s, generator=g, dtype=dt)

    def put(case, **kw):
        for k, v in kw.items():
            out["%s/%s" % (case, k)] = _np(v) if isinstance(v, torch.Tensor) else np.asarray(v)

    B, Cin, Cout, IH, IW, OH, OW, K, P = 2, 3, 5, 7, 9, 6, 8, 4, 3
    for dt, dn in ((torch.float32, "f32"), (torch.float64, "f64")):
        span = torch.tensor([IW + 3.0, IH + 3.0], dtype=dt)
        for interp in (0, 1, 2):
            for weighted in (False, True):
                tag = "%s_i%d_%s" % (dn, interp, "w" if weighted else "u")
                x = rnd(B, Cin, IH, IW, dt=dt)
                w = rnd(Cout, Cin, K, dt=dt)
                b = rnd(Cout, dt=dt)
                gy = rnd(B, Cout, OH, OW, dt=dt)
                if weighted:
                    m = uni(OH, OW, K, P, 2, dt=dt) * span - 1.5
                    iw = uni(OH, OW, K, P, dt=dt)
                    m1, iw1 = m[:, :, 0].contiguous(), iw[:, :, 0].contiguous()
                else:
                    m = uni(OH, OW, K, 2, dt=dt) * span - 1.5
                    iw = None
                    m1, iw1 = m[:, :, 0].contiguous(), None
                base = dict(interp=interp, K=K, sample_map=m)
                if weighted:
                    base["interp_weights"] = iw

                # conv
                if weighted:
                    y = R.weighted_mapped_conv_forward(x, m, iw, w, b, K, interp)
                    gx, gw, gb = R.weighted_mapped_conv_backward(gy, m, iw, x, w, b, K, interp)
                else:
                    y = R.mapped_conv_forward(x, m, w, b, K, interp)
                    gx, gw, gb = R.mapped_conv_backward(gy, m, x, w, b, K, interp)
                put("conv_" + tag, input=x, weight=w, bias=b, grad_output=gy, output=y,
                    grad_input=gx, grad_weight=gw, grad_bias=gb, **base)

                # transposed conv: x on the (OH, OW) grid, output (IH, IW)
                xt = rnd(B, Cin, OH, OW, dt=dt)
                wt = rnd(Cin, Cout, K, dt=dt)
                gyt = rnd(B, Cout, IH, IW, dt=dt)
                if weighted:
                    yt = R.weighted_mapped_transposed_conv_forward(xt, m, iw, wt, b, IH, IW, K, interp)
                    tgx, tgw, tgb = R.weighted_mapped_transposed_conv_backward(gyt, m, iw, xt, wt, b,
                                                                               K, interp)
                else:
                    yt = R.mapped_transposed_conv_forward(xt, m, wt, b, IH, IW, K, interp)
                    tgx, tgw, tgb = R.mapped_transposed_conv_backward(gyt, m, xt, wt, b, K, interp)
                put("tconv_" + tag, input=xt, weight=wt, bias=b, grad_output=gyt, output=yt,
                    grad_input=tgx, grad_weight=tgw, grad_bias=tgb, oh=IH, ow=IW, **base)

                # pooling.  Inputs are positive so that the start value of the running maximum
                # (which differs between the reference's CPU and CUDA builds) never matters.
                xp = uni(B, Cin, IH, IW, dt=dt) + 0.5
                gp = rnd(B, Cin, OH, OW, dt=dt)
                # tap 0 always lies inside the image, so every window has a positive maximum and
                # the reference CPU build never emits index -1 (which its unpool would read as an
                # out-of-bounds map offset)
                inside = torch.tensor([IW - 1.4, IH - 1.4], dtype=dt)
                m = m.clone()
                m[:, :, 0] = uni(*m[:, :, 0].shape, dt=dt) * inside + 0.2
                base = dict(base, sample_map=m)
                if weighted:
                    # weights bounded away from zero keep every tap value positive or exactly zero
                    mp_, idx = R.weighted_mapped_max_pool(xp, m, iw, K, interp)
                    mu = R.weighted_mapped_max_unpool(gp, idx, m, iw, IH, IW, K, interp)
                    ap = R.weighted_mapped_avg_pool(x, m, iw, K, interp)
                    au = R.weighted_mapped_avg_unpool(gp, m, iw, IH, IW, K, interp)
                else:
                    mp_, idx = R.mapped_max_pool(xp, m, K, interp)
                    mu = R.mapped_max_unpool(gp, idx, m, IH, IW, K, interp)
                    ap = R.mapped_avg_pool(x, m, K, interp)
                    au = R.mapped_avg_unpool(gp, m, IH, IW, K, interp)
                put("pool_" + tag, input=x, input_pos=xp, grad_output=gp, max_output=mp_,
                    max_idx=idx, max_unpool=mu, avg_output=ap, avg_unpool=au, **base)

                # resample
                xg = rnd(B, Cin, OH, OW, dt=dt)
                if weighted:
                    ga = R.weighted_resample_from_map(x, m1, iw1, interp)
                    sc = R.weighted_resample_to_map(xg, m1, iw1, IH, IW, interp)
                else:
                    ga = R.resample_from_map(x, m1, interp)
                    sc = R.resample_to_map(xg, m1, IH, IW, interp)
                rs = dict(interp=interp, sample_map=m1)
                if weighted:
                    rs["interp_weights"] = iw1
                put("resample_" + tag, input=x, gather_output=ga, grid_input=xg, scatter_output=sc,
                    oh=IH, ow=IW, **rs)

    # max pool on N(0,1) data with the reference CPU build's start value (smallest positive
    # normal): outputs with index -1 mark windows whose taps were all <= that value
    x = rnd(2, 4, 6, 7, dt=torch.float32)
    m = uni(5, 6, 3, 2, dt=torch.float32) * torch.tensor([9.0, 8.0]) - 1.0
    y, idx = R.mapped_max_pool(x, m, 3, 0)
    put("pool_cpu_init_f32", input=x, sample_map=m, K=3, interp=0, max_output=y, max_idx=idx)
    return out


def config1():
    """float32, batch 1, 3 -> 16 channels, 64 x 128, K = 9: a regular 3x3 grid around each output
    pixel plus U(-0.5, 0.5) jitter, bilinear.  Draw order after manual_seed(0): x, w, bias, jitter,
    then the upstream gradient."""
    R = ref.ops()
    torch.manual_seed(0)
    H, W, K = 64, 128, 9
    x = torch.randn(1, 3, H, W)
    w = torch.randn(16, 3, K)
    b = torch.randn(16)
    jit = torch.rand(H, W, K, 2) - 0.5
    gy = torch.randn(1, 16, H, W)
    ys, xs = torch.meshgrid(torch.arange(H, dtype=torch.float32),
                            torch.arange(W, dtype=torch.float32), indexing="ij")
    dy, dx = torch.meshgrid(torch.tensor([-1.0, 0.0, 1.0]), torch.tensor([-1.0, 0.0, 1.0]),
                            indexing="ij")
    m = torch.stack([xs[..., None] + dx.reshape(-1), ys[..., None] + dy.reshape(-1)], -1) + jit
    m = m.contiguous()
    y = R.mapped_conv_forward(x, m, w, b, K, 1)
    gx, gw, gb = R.mapped_conv_backward(gy, m, x, w, b, K, 1)
    return {"input": _np(x), "weight": _np(w), "bias": _np(b), "sample_map": _np(m),
            "grad_output": _np(gy), "output": _np(y), "grad_input": _np(gx), "grad_weight": _np(gw),
            "grad_bias": _np(gb), "K": np.asarray(K), "interp": np.asarray(1)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get(
        "MC_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference")))
    a = ap.parse_args()
    assert ref.available(), "build the reference CPU extensions first: python oracle/build_ref.py"
    kats, n = capture_kats(a.ref)
    np.savez_compressed(os.path.join(HERE, "kat.npz"), **kats)
    print("%d reference CPU known-answer tests passed and recorded" % n)
    np.savez_compressed(os.path.join(HERE, "random_small.npz"), **random_cases())
    np.savez_compressed(os.path.join(HERE, "config1.npz"),
                        **{"config1/" + k: v for k, v in config1().items()})
    for f in ("kat.npz", "random_small.npz", "config1.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
