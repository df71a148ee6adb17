from mappedconvolutions_b200.host import impl as _impl

knn_forward = _impl.knn_forward
