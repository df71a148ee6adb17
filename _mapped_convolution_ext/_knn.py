from mappedconvolutions_b200.ops import knn_forward  # noqa: F401
