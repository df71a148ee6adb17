from mappedconvolutions_b200.ops import weighted_mapped_max_pool, weighted_mapped_max_unpool  # noqa: F401
