from mappedconvolutions_b200.ops import resample_to_map, resample_from_map  # noqa: F401
