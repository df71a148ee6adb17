"""Loader for the reference's own CPU extensions built by oracle/build_ref.py (checker only).

`ops()` returns a namespace with the reference's pybind functions (mapped_conv_forward, ...),
all running the reference's unmodified CPU code.  Nothing in the product package imports this.
"""
import importlib.machinery
import importlib.util
import os
import types

HERE = os.path.dirname(os.path.abspath(__file__))
EXT_DIR = os.path.join(HERE, "_ref", "_mapped_convolution_ext")

_MODS = ["_mapped_convolution", "_mapped_transposed_convolution", "_mapped_max_pooling",
         "_mapped_avg_pooling", "_resample", "_weighted_mapped_convolution",
         "_weighted_mapped_transposed_convolution", "_weighted_mapped_max_pooling",
         "_weighted_mapped_avg_pooling", "_weighted_resample"]
_cache = {}


def available():
    return all(os.path.exists(os.path.join(EXT_DIR, m + ".so")) for m in _MODS)


def load(name):
    """Import one built reference module by file path."""
    if name not in _cache:
        import torch  # noqa: F401  (the extension links against libtorch)
        path = os.path.join(EXT_DIR, name + ".so")
        loader = importlib.machinery.ExtensionFileLoader(name, path)
        spec = importlib.util.spec_from_file_location(name, path, loader=loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
        _cache[name] = mod
    return _cache[name]


def ops():
    ns = types.SimpleNamespace()
    for m in _MODS:
        mod = load(m)
        for k in dir(mod):
            if not k.startswith("_"):
                setattr(ns, k, getattr(mod, k))
    return ns
