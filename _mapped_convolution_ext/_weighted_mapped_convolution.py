from mappedconvolutions_b200.ops import weighted_mapped_conv_forward, weighted_mapped_conv_backward  # noqa: F401
