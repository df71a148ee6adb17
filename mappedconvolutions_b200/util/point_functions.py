from ..host import impl as ops


def knn(ref, query, k):
    """k nearest reference points of every query point.

    ref (B, D, M), query (B, D, N) float32 CUDA tensors -> (idx (B, k, N) int64, dist (B, k, N)),
    nearest first, ties by lower index.  Indices are 1-based, as the reference's kernel writes
    them (include/util/cuda/knn.cuh:141,160,184); package/layers/util/point_functions.py:7-17.
    """
    return ops.knn_forward(ref, query, k)
