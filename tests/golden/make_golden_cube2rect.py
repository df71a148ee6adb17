"""Generate tests/golden/cube2rect_ref.npz by running the REFERENCE's own CUDA cube2rect
(oracle/_ref/_mapped_convolution_ext/_cube2rect.so, built from the reference's sources for sm_100a
by `python oracle/build_ref.py --cube2rect`) on a GPU: the reference has no CPU version of this op.

The kernel's bilinear branch may read the element that follows the cube map (the right neighbour
of the last face's last pixel, with weight zero: include/util/cuda/cube2rect.cuh:46-62 hands the
sampler the whole 6 * cube_dim row as width), so every cube map here is a view into a larger zeroed
buffer.

    python tests/golden/make_golden_cube2rect.py <output.npz>
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import ref  # noqa: E402

# name: channels, cube_dim, rect_h, rect_w, dtype
CASES = {
    "c3_d8_16x32_f32": (3, 8, 16, 32, torch.float32),
    "c1_d16_33x64_f32": (1, 16, 33, 64, torch.float32),     # odd height: a row on the equator
    "c2_d5_20x41_f64": (2, 5, 20, 41, torch.float64),
    "c4_d32_64x128_f32": (4, 32, 64, 128, torch.float32),
    "c1_d2_9x16_f32": (1, 2, 9, 16, torch.float32),         # two-pixel faces: every sample near an edge
}


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "cube2rect_ref.npz")
    fn = ref.load("_cube2rect").cube2rect
    g = torch.Generator().manual_seed(0)
    out = {}
    for name, (C, D, RH, RW, dt) in CASES.items():
        cube = torch.randn(C, D, 6 * D, generator=g, dtype=dt)
        buf = torch.zeros(C * D * 6 * D + 64, dtype=dt, device="cuda")
        dev = buf[:C * D * 6 * D].view(C, D, 6 * D)
        dev.copy_(cube)
        out[name + "/cube"] = cube.numpy()
        out[name + "/shape"] = np.array([RH, RW], dtype=np.int64)
        for interp, tag in ((0, "nearest"), (1, "bilinear")):
            rect = fn(dev, RH, RW, interp)
            torch.cuda.synchronize()
            out[name + "/" + tag] = rect.cpu().numpy()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, "with", len(CASES), "cases")


if __name__ == "__main__":
    main()
