"""Module names of the reference's compiled extension package (package/setup.py:51-95), each
re-exporting the functions of the same names from the compiled host binding
(mappedconvolutions_b200.host: the PyTorch C++ extension, or its ctypes twin when that is not built)."""
