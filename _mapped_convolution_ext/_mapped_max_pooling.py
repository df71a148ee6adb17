from mappedconvolutions_b200.ops import mapped_max_pool, mapped_max_unpool  # noqa: F401
