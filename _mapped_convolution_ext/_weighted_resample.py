from mappedconvolutions_b200.ops import weighted_resample_to_map, weighted_resample_from_map  # noqa: F401
