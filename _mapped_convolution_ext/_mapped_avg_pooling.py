from mappedconvolutions_b200.host import impl as _impl

mapped_avg_pool = _impl.mapped_avg_pool
mapped_avg_unpool = _impl.mapped_avg_unpool
