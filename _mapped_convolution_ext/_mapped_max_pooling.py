from mappedconvolutions_b200.host import impl as _impl

mapped_max_pool = _impl.mapped_max_pool
mapped_max_unpool = _impl.mapped_max_unpool
