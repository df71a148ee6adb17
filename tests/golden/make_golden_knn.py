"""Generate tests/golden/knn_ref.npz by running the REFERENCE's own CUDA k-NN
(oracle/_ref/_mapped_convolution_ext/_knn.so, built from the reference's sources for sm_100a by
`python oracle/build_ref.py --knn`) on a GPU.

The reference allocates a (k, N) buffer and uses it as the (M, N) distance matrix
(src/util/cuda/knn_layer.cu:20-23; include/util/cuda/knn.cuh:111-112 writes rows < M, :144-187
reads rows < max(k, M)), so it is in bounds exactly when M == k: every case here has M == k, which
is asserted before each call.  With M == k the kernel still computes every distance with its own
arithmetic, sorts all of them with its insertion sort (ordering and tie-breaks), numbers them from 1
and takes the square roots - the behaviours the library's k-NN must reproduce bit for bit.

    python tests/golden/make_golden_knn.py <output.npz>
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import ref  # noqa: E402


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "knn_ref.npz")
    knn = ref.load("_knn").knn_forward
    g = torch.Generator().manual_seed(0)
    out = {}
    cases = [("k9_d3", 2, 3, 9, 200), ("k16_d3", 1, 3, 16, 256), ("k32_d5", 1, 5, 32, 77),
             ("k9_d5_dup", 1, 5, 9, 64), ("k16_d3_sphere", 1, 3, 16, 128), ("k12_d16", 1, 16, 12, 40)]
    for name, B, D, k, N in cases:
        refp = torch.randn(B, D, k, generator=g)
        query = torch.randn(B, D, N, generator=g)
        if "dup" in name:          # exact duplicates among the reference points: ties by index
            refp[:, :, 5] = refp[:, :, 2]
            refp[:, :, 7] = refp[:, :, 2]
            query[:, :, :8] = refp[:, :, :8]
        if "sphere" in name:       # unit vectors, query = a subset of the references (distance 0)
            refp = refp / refp.norm(dim=1, keepdim=True)
            query = query / query.norm(dim=1, keepdim=True)
            query[:, :, :k] = refp
        M = refp.shape[2]
        assert M == k, "the reference's k-NN is only in bounds for M == k"
        idx, dist = knn(refp.cuda().contiguous(), query.cuda().contiguous(), k)
        torch.cuda.synchronize()
        out[name + "/ref"], out[name + "/query"] = refp.numpy(), query.numpy()
        out[name + "/k"] = np.int64(k)
        out[name + "/idx"], out[name + "/dist"] = idx.cpu().numpy(), dist.cpu().numpy()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, "with", len(cases), "cases")


if __name__ == "__main__":
    main()
