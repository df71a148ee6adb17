from mappedconvolutions_b200.host import impl as _impl

cube2rect = _impl.cube2rect
