from mappedconvolutions_b200.host import impl as _impl

weighted_mapped_avg_pool = _impl.weighted_mapped_avg_pool
weighted_mapped_avg_unpool = _impl.weighted_mapped_avg_unpool
