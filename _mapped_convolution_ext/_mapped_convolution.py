from mappedconvolutions_b200.host import impl as _impl

mapped_conv_forward = _impl.mapped_conv_forward
mapped_conv_backward = _impl.mapped_conv_backward
