from mappedconvolutions_b200.host import impl as _impl

resample_to_map = _impl.resample_to_map
resample_from_map = _impl.resample_from_map
