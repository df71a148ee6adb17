from mappedconvolutions_b200.host import impl as _impl

weighted_mapped_max_pool = _impl.weighted_mapped_max_pool
weighted_mapped_max_unpool = _impl.weighted_mapped_max_unpool
