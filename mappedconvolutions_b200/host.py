"""Host binding behind the layer API and the reference's pybind module names.

`impl` is the compiled PyTorch C++ extension (`_mc_torch_ext`, csrc_torch/mc_torch_ext.cpp, built
in-tree by `build.build_torch_ext`) when it is present, otherwise its ctypes twin `ops`.  Both
carry the reference's function names and call the same C ABI; neither has a CPU path.
"""
try:
    from . import _mc_torch_ext as impl
    COMPILED = True
except ImportError:  # not built (no host compiler at hand): same logic on ctypes
    from . import ops as impl
    COMPILED = False
