from mappedconvolutions_b200.ops import mapped_transposed_conv_forward, mapped_transposed_conv_backward  # noqa: F401
