"""ctypes binding of the C-ABI library (include/mc_b200.h).

The library is the only compute path: if it cannot be loaded the import of any op fails loudly;
there is no CPU or PyTorch fallback.
"""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libmc_b200.so")

MC_F32, MC_F64, MC_BF16 = 0, 1, 2
MC_NCHW, MC_NHWC = 0, 1
MC_FLAG_RELU = 1


class McDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in
                ("B", "C_in", "C_out", "IH", "IW", "OH", "OW", "K", "P", "interp", "dtype", "layout",
                 "flags")]


class McError(RuntimeError):
    pass


_lib = None

_vp, _sz, _i32 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int32
_dp = ctypes.POINTER(McDesc)

# name -> (restype, argtypes); mirrors include/mc_b200.h declaration by declaration
SIGNATURES = {
    "mc_strerror": (ctypes.c_char_p, [ctypes.c_int]),
    "mc_abi_version": (ctypes.c_int, []),
    "mc_kernel_launch_count": (ctypes.c_uint64, []),
    "mc_device_status": (ctypes.c_int, [_vp, ctypes.c_int]),
    "mc_selftest_wait_expiry": (ctypes.c_int, [_vp, _vp]),
    "mc_conv_fwd": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mc_conv_fwd_workspace_bytes": (_sz, [_dp]),
    "mc_conv_fwd_static_scratch_limit": (_sz, []),
    "mc_conv_fwd_static_scratch": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mc_conv_dgrad": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mc_conv_dgrad_workspace_bytes": (_sz, [_dp]),
    "mc_tapmap_bytes": (_sz, [_dp]),
    "mc_tapmap_build": (ctypes.c_int, [_dp, _vp, _vp, _sz, _vp]),
    "mc_conv_fwd_tap": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mc_conv_wgrad_tap": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mc_invmap_bytes": (_sz, [_dp]),
    "mc_invmap_build_workspace_bytes": (_sz, [_dp]),
    "mc_invmap_build": (ctypes.c_int, [_dp, _vp, _vp, _sz, _vp, _sz, _vp]),
    "mc_conv_dgrad_inv_supported": (ctypes.c_int, [_dp]),
    "mc_conv_dgrad_inv_workspace_bytes": (_sz, [_dp]),
    "mc_conv_dgrad_inv": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mc_conv_dgrad_tapsum": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp]),
    "mc_rowplan_analysis_bytes": (_sz, [_dp]),
    "mc_rowplan_analyse": (ctypes.c_int, [_dp, _vp, _vp, _vp]),
    "mc_rowplan_assemble": (ctypes.c_int64, [_dp, _vp, _vp, _vp, ctypes.c_int64]),
    "mc_conv_rowplan_workspace_bytes": (_sz, [_dp, _vp, _i32]),
    "mc_conv_fwd_rowplan": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mc_conv_dgrad_rowplan": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mc_conv_wgrad_rowplan_workspace_bytes": (_sz, [_dp, _vp]),
    "mc_conv_wgrad_rowplan": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mc_conv_wgrad": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mc_conv_wgrad_workspace_bytes": (_sz, [_dp]),
    "mc_tconv_fwd": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mc_tconv_dgrad": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mc_tconv_wgrad": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mc_tconv_workspace_bytes": (_sz, [_dp]),
    "mc_bias_grad": (ctypes.c_int, [_dp, _vp, _vp, _vp]),
    "mc_pool_max_fwd": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mc_pool_max_bwd": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mc_pool_avg_fwd": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp]),
    "mc_pool_avg_bwd": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mc_scatter_workspace_bytes": (_sz, [_dp]),
    "mc_pool_avg_bwd_inv": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp]),
    "mc_resample_scatter_inv": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp]),
    "mc_resample_gather": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp]),
    "mc_resample_scatter": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mc_knn": (ctypes.c_int, [_vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp]),
    "mc_sphere_locate": (ctypes.c_int, [_vp, ctypes.c_int64, _i32, ctypes.POINTER(_vp),
                                        ctypes.POINTER(_vp), ctypes.POINTER(_vp),
                                        ctypes.POINTER(_i32), _i32, _vp, _vp, _vp, _vp]),
    "mc_conv_wgrad_tap_relu": (ctypes.c_int, [_dp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mc_weighted_plan_desc": (ctypes.c_int, [_dp, _dp]),
    "mc_tapmap_build_weighted": (ctypes.c_int, [_dp, _vp, _vp, _vp, _sz, _vp]),
    "mc_invmap_build_weighted": (ctypes.c_int, [_dp, _vp, _vp, _vp, _sz, _vp, _sz, _vp]),
    "mc_cube2rect": (ctypes.c_int, [_i32, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp]),
    "mc_voting_resample_workspace": (_sz, [_i32, _i32, _i32, _i32, _i32]),
    "mc_voting_resample": (ctypes.c_int, [_vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _sz,
                                          _vp, _vp]),
}


def lib():
    """Return the loaded library, loading it on first use."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise McError(
                "CUDA library %s is missing; build it with "
                "`python -m mappedconvolutions_b200.build` (there is no fallback path)" % LIB_PATH)
        h = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(h, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = h
    return _lib


def check(code):
    if code != 0:
        raise McError("mc_b200: %s (code %d)" % (lib().mc_strerror(code).decode(), code))
