from mappedconvolutions_b200.ops import mapped_avg_pool, mapped_avg_unpool  # noqa: F401
