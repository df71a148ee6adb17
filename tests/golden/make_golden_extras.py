"""Generate tests/golden/extras.npz from the REFERENCE's own CPU code:

  vote/*   voting-resample vectors (oracle/_ref/_mapped_convolution_ext/_voting_resample.so, built
           from the reference's sources by `python oracle/build_ref.py`);
  grid/*   the reference's plain grid `Convolution` / `TransposedConvolution` layers
           (package/layers/nn/convolution_layer.py, transposed_convolution_layer.py on top of the
           reference's _convolution / _transposed_convolution CPU extensions): parameters after
           `torch.manual_seed(0)`, output and gradients on a seeded input.

    python tests/golden/make_golden_extras.py [output.npz] [--ref /path/to/reference]
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import ref  # noqa: E402

# name: B, C, IH, IW, OH, OW, candidates
CASES = {
    "labels_1ch": (2, 1, 24, 48, 8, 16, 13),       # a label image reduced 3 x: several votes per pixel
    "labels_3ch": (2, 3, 9, 11, 4, 5, 7),          # channels share the vote table (see the oracle)
    "sparse": (1, 1, 6, 7, 20, 20, 5),             # most target pixels get no vote -> label 0
    "one_pixel": (3, 2, 17, 5, 1, 1, 40),          # every vote lands on one pixel
    "outside": (1, 1, 12, 12, 6, 6, 4),            # a third of the targets lie outside the image
}


def make_case(name, g):
    B, C, IH, IW, OH, OW, NC = CASES[name]
    labels = torch.randint(0, NC, (B, C, IH, IW), generator=g)
    lo = -3 if name == "outside" else 0
    mx = torch.randint(lo, OW - lo, (IH, IW), generator=g)
    my = torch.randint(lo, OH - lo, (IH, IW), generator=g)
    if name == "labels_1ch":   # nearest-neighbour reduction with a little jitter: realistic ties
        yy, xx = torch.meshgrid(torch.arange(IH), torch.arange(IW), indexing="ij")
        mx, my = xx // 3, yy // 3
        labels = ((xx // 5 + yy // 4) % NC).expand(B, C, IH, IW).clone()
        noise = torch.rand(B, C, IH, IW, generator=g) < 0.2
        labels[noise] = torch.randint(0, NC, (int(noise.sum()),), generator=g)
    return labels.contiguous(), torch.stack([mx, my], -1).contiguous()


# name: layer class, constructor arguments, input shape
GRID_CASES = {
    "conv_3x3_p1": ("Convolution", dict(in_channels=3, out_channels=5, kernel_size=3, padding=1), (2, 3, 7, 9)),
    "conv_3x2_s2_d2": ("Convolution", dict(in_channels=4, out_channels=2, kernel_size=(3, 2), stride=2, padding=(2, 1),
                                           dilation=(2, 1)), (1, 4, 11, 8)),
    "tconv_2x2_s2": ("TransposedConvolution", dict(in_channels=3, out_channels=4, kernel_size=2, stride=2), (2, 3, 5, 6)),
    "tconv_3x3_p1_d2": ("TransposedConvolution", dict(in_channels=2, out_channels=3, kernel_size=3, padding=1,
                                                      dilation=2), (1, 2, 6, 5)),
}


def reference_grid_layers(ref_root):
    """The reference's two grid layer classes, loaded from its checkout with its CPU extensions."""
    ext = types.ModuleType("_mapped_convolution_ext")
    ext._convolution = ref.load("_convolution")
    ext._transposed_convolution = ref.load("_transposed_convolution")
    sys.modules.update({"_mapped_convolution_ext": ext, "_mapped_convolution_ext._convolution": ext._convolution,
                        "_mapped_convolution_ext._transposed_convolution": ext._transposed_convolution})
    pkg = types.ModuleType("refnn")
    pkg.__path__ = [os.path.join(ref_root, "package", "layers", "nn")]
    sys.modules["refnn"] = pkg
    mods = {}
    for name in ("layer_utils", "convolution_layer", "transposed_convolution_layer"):
        spec = importlib.util.spec_from_file_location("refnn." + name, os.path.join(pkg.__path__[0], name + ".py"))
        mods[name] = importlib.util.module_from_spec(spec)
        sys.modules["refnn." + name] = mods[name]
        spec.loader.exec_module(mods[name])
    return {"Convolution": mods["convolution_layer"].Convolution,
            "TransposedConvolution": mods["transposed_convolution_layer"].TransposedConvolution}


def main():
    args = [a for a in sys.argv[1:]]
    ref_root = os.environ.get("MC_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))
    if "--ref" in args:
        i = args.index("--ref")
        ref_root = args[i + 1]
        del args[i:i + 2]
    out_path = args[0] if args else os.path.join(HERE, "extras.npz")
    vote = ref.load("_voting_resample").voting_resample_to_map
    g = torch.Generator().manual_seed(0)
    out = {}
    for name, (B, C, IH, IW, OH, OW, NC) in CASES.items():
        labels, smap = make_case(name, g)
        res = vote(labels.clone(), smap.clone(), OH, OW, NC)
        out["vote/%s/labels" % name], out["vote/%s/map" % name] = labels.numpy(), smap.numpy()
        out["vote/%s/args" % name] = np.array([OH, OW, NC], dtype=np.int64)
        out["vote/%s/out" % name] = res.numpy()
    layers = reference_grid_layers(ref_root)
    for name, (cls, kw, shape) in GRID_CASES.items():
        torch.manual_seed(0)
        layer = layers[cls](**kw)
        x = torch.randn(*shape, generator=g, requires_grad=True)
        y = layer(x)
        gy = torch.randn(y.shape, generator=g)
        y.backward(gy)
        for k, v in (("weight", layer.weight), ("bias", layer.bias), ("x", x), ("y", y), ("gy", gy), ("gx", x.grad),
                     ("gw", layer.weight.grad), ("gb", layer.bias.grad)):
            out["grid/%s/%s" % (name, k)] = v.detach().numpy()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, "with", len(CASES), "voting and", len(GRID_CASES), "grid-layer cases")


if __name__ == "__main__":
    main()
