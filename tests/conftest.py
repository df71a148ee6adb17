import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


# The op surface exists twice: the compiled PyTorch C++ extension (what the layer API and the
# benchmark call) and its ctypes twin.  The GPU parity tests of these modules run once against
# each; they import the surface as `from mappedconvolutions_b200 import ops`, which this fixture
# points at the binding under test.
_TWO_BINDINGS = {"test_gpu_parity", "test_gpu_kat"}
_COMPILED_ONLY = {"test_gpu_full_size"}


def pytest_generate_tests(metafunc):
    name = metafunc.module.__name__
    if name in _TWO_BINDINGS:
        metafunc.parametrize("op_binding", ["ctypes", "compiled"], indirect=True)
    elif name in _COMPILED_ONLY:
        metafunc.parametrize("op_binding", ["compiled"], indirect=True)


@pytest.fixture(autouse=True)
def op_binding(request, monkeypatch):
    which = getattr(request, "param", None)
    if which == "compiled":
        import mappedconvolutions_b200
        from mappedconvolutions_b200 import host
        assert host.COMPILED, "extension not built: python -m mappedconvolutions_b200.build"
        monkeypatch.setattr(mappedconvolutions_b200, "ops", host.impl)
    return which
