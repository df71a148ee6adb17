from mappedconvolutions_b200.ops import weighted_mapped_avg_pool, weighted_mapped_avg_unpool  # noqa: F401
