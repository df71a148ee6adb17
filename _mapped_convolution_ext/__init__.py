"""Module names of the reference's compiled extension package (package/setup.py:51-95), each
re-exporting the functions of mappedconvolutions_b200.ops that carry the same names."""
