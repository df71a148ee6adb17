from mappedconvolutions_b200.host import impl as _impl

weighted_resample_to_map = _impl.weighted_resample_to_map
weighted_resample_from_map = _impl.weighted_resample_from_map
