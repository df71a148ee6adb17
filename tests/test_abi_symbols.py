"""CPU: the C-ABI library loads and exports every entry point that include/mc_b200.h declares,
and the ctypes binding table covers each of them.  No compute call is made."""
import ctypes
import os
import re

import pytest

from mappedconvolutions_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    src = open(os.path.join(ROOT, "include", "mc_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(mc_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for must in ("mc_conv_fwd", "mc_conv_dgrad", "mc_conv_wgrad", "mc_tconv_fwd", "mc_pool_max_fwd",
                 "mc_pool_avg_bwd", "mc_resample_gather", "mc_resample_scatter", "mc_knn"):
        assert must in syms


def test_library_exports_every_declared_symbol():
    if not os.path.exists(_lib.LIB_PATH):
        from mappedconvolutions_b200 import build
        build.build()
    h = ctypes.CDLL(_lib.LIB_PATH)
    for s in declared_symbols():
        assert hasattr(h, s), "libmc_b200.so does not export " + s


def test_binding_table_matches_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_error_strings_and_version():
    L = _lib.lib()
    assert L.mc_abi_version() >= 1
    assert L.mc_strerror(0) == b"ok"
    for code in range(-6, 0):
        assert len(L.mc_strerror(code)) > 3
    with pytest.raises(_lib.McError):
        _lib.check(-1)


def test_bad_descriptor_is_rejected_without_a_gpu():
    """Argument validation happens before any CUDA call, so it can be exercised on a CPU box."""
    L = _lib.lib()
    d = _lib.McDesc(0, 1, 1, 4, 4, 4, 4, 1, 0, 1, 0, 0)  # B = 0
    assert L.mc_conv_fwd(d, None, None, None, None, None, None, None, 0, None) == -1
    d = _lib.McDesc(1, 1, 1, 4, 4, 4, 4, 1, 0, 1, 0, 0)
    assert L.mc_conv_fwd(d, None, None, None, None, None, None, None, 0, None) == -1  # null x
    assert L.mc_knn(None, None, 1, 3, 8, 8, 4, None, None, None) == -1
    d = _lib.McDesc(1, 1, 1, 4, 4, 4, 4, 2, 0, 1, 0, 0)  # resample needs K == 1
    assert L.mc_resample_gather(d, 1, 1, None, 1, None) == -1
