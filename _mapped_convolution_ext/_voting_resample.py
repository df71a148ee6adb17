from mappedconvolutions_b200.host import impl as _impl

voting_resample_to_map = _impl.voting_resample_to_map
