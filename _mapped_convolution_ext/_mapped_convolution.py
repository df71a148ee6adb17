from mappedconvolutions_b200.ops import mapped_conv_forward, mapped_conv_backward  # noqa: F401
