"""opscv_b200: ctypes caller of libopscv_b200.so, the B200 implementation of the ops-cv resampling aclnn API.

The product is the shared library (C ABI declared in include/aclnn_resample.h and include/opscv_acl.h). This
package is the thin Python caller used by the tests and the benchmark, playing the part that the reference's
ATK `pyaclnn` backend plays for the original library: it builds aclTensor handles over torch CUDA tensors
(device memory and streams only), runs the two-phase calls and raises on any non-zero status. It contains no
arithmetic and no fallback: if the library is missing, loading fails.

The directory name has a hyphen, so import it through `__graft_entry__.load_package()` (registers it as the
module `opscv_b200`).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libopscv_b200.so")
CSRC_DIR = os.path.join(_HERE, "csrc")

# aclDataType / aclFormat values (include/opscv_acl.h)
ACL_FLOAT, ACL_FLOAT16, ACL_INT8, ACL_INT32, ACL_UINT8, ACL_INT64, ACL_DOUBLE, ACL_BOOL, ACL_BF16 = 0, 1, 2, 3, 4, 9, 11, 12, 27
ACL_FORMAT_NCHW, ACL_FORMAT_NHWC, ACL_FORMAT_ND, ACL_FORMAT_NCL = 0, 1, 2, 47
ACL_FORMAT_NDHWC, ACL_FORMAT_NCDHW = 27, 30
ACL_OPT_DETERMINISTIC = 0

ACLNN_SUCCESS = 0
ACLNN_ERR_PARAM_NULLPTR = 161001
ACLNN_ERR_PARAM_INVALID = 161002
ACLNN_ERR_RUNTIME_ERROR = 361001
ACLNN_ERR_INNER_NULLPTR = 561103

# Every symbol include/*.h declares, with (restype, argtypes). Used to bind and, in the CPU tests, to check that
# the library exports all of them.
_P, _U64, _I64, _I32, _F, _D, _B = (ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int64, ctypes.c_int32, ctypes.c_float,
                                    ctypes.c_double, ctypes.c_bool)
_PU64, _PP = ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_void_p)
_PHASE2 = (_I32, [_P, _U64, _P, _P])
SYMBOLS = {
    "aclCreateTensor": (_P, [ctypes.POINTER(_I64), _U64, _I32, ctypes.POINTER(_I64), _I64, _I32,
                             ctypes.POINTER(_I64), _U64, _P]),
    "aclDestroyTensor": (_I32, [_P]),
    "aclCreateIntArray": (_P, [ctypes.POINTER(_I64), _U64]),
    "aclDestroyIntArray": (_I32, [_P]),
    "aclCreateBoolArray": (_P, [ctypes.POINTER(_B), _U64]),
    "aclDestroyBoolArray": (_I32, [_P]),
    "aclCreateFloatArray": (_P, [ctypes.POINTER(_F), _U64]),
    "aclDestroyFloatArray": (_I32, [_P]),
    "aclGetFloatArraySize": (_I32, [_P, _PU64]),
    "aclDestroyAclOpExecutor": (_I32, [_P]),
    "aclGetRecentErrMsg": (ctypes.c_char_p, []),
    "aclrtCtxSetSysParamOpt": (ctypes.c_int, [_I32, _I64]),
    "aclrtCtxGetSysParamOpt": (ctypes.c_int, [_I32, ctypes.POINTER(_I64)]),
    "opscvSetBackwardAlgo": (_I32, [_I32]),
    "opscvGetBackwardAlgo": (_I32, []),
    "opscvVersion": (_I32, []),
    "opscvGetLaunchCount": (_U64, []),
    "opscvResetLaunchCount": (None, []),
    "opscvGetAsyncCopyTimeouts": (ctypes.c_uint32, []),
    "opscvDebugAxisTable": (_I32, [_I32, _I64, _I64, _I32, _F, _P, _P, _P, ctypes.POINTER(_I32)]),
    "opscvUpsampleBilinear2dNoAlloc": (_I32, [_P, _P, _I32, _I32, _I64, _I64, _I64, _I64, _I64, _I64, _B, _D, _D, _P]),
    "aclnnUpsampleNearest2dGetWorkspaceSize": (_I32, [_P, _P, _P, _PU64, _PP]),
    "aclnnUpsampleNearest2d": _PHASE2,
    "aclnnUpsampleNearest2dV2GetWorkspaceSize": (_I32, [_P, _P, _F, _F, _P, _PU64, _PP]),
    "aclnnUpsampleNearest2dV2": _PHASE2,
    "aclnnUpsampleNearest2dBackwardGetWorkspaceSize": (_I32, [_P, _P, _P, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleNearest2dBackward": _PHASE2,
    "aclnnUpsampleBilinear2dGetWorkspaceSize": (_I32, [_P, _P, _B, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleBilinear2d": _PHASE2,
    "aclnnUpsampleBilinear2dBackwardGetWorkspaceSize": (_I32, [_P, _P, _P, _B, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleBilinear2dBackward": _PHASE2,
    "aclnnUpsampleBilinear2dBackwardV2GetWorkspaceSize": (_I32, [_P, _P, _P, _B, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleBilinear2dBackwardV2": _PHASE2,
    "aclnnUpsampleBicubic2dAAGetWorkspaceSize": (_I32, [_P, _P, _B, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleBicubic2dAA": _PHASE2,
    "aclnnUpsampleBicubic2dAAGradGetWorkspaceSize": (_I32, [_P, _P, _P, _B, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleBicubic2dAAGrad": _PHASE2,
    "aclnnUpsampleNearestExact2dGetWorkspaceSize": (_I32, [_P, _P, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleNearestExact2d": _PHASE2,
    "aclnnUpsampleNearestExact2dBackwardGetWorkspaceSize": (_I32, [_P, _P, _P, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleNearestExact2dBackward": _PHASE2,
    "aclnnUpsampleNearestExact1dGetWorkspaceSize": (_I32, [_P, _P, _D, _P, _PU64, _PP]),
    "aclnnUpsampleNearestExact1d": _PHASE2,
    "aclnnUpsampleNearestExact1dBackwardGetWorkspaceSize": (_I32, [_P, _P, _P, _D, _P, _PU64, _PP]),
    "aclnnUpsampleNearestExact1dBackward": _PHASE2,
    "aclnnUpsampleBilinear2dAAGetWorkspaceSize": (_I32, [_P, _P, _B, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleBilinear2dAA": _PHASE2,
    "aclnnUpsampleBilinear2dAABackwardGetWorkspaceSize": (_I32, [_P, _P, _P, _B, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleBilinear2dAABackward": _PHASE2,
    "aclnnUpsampleBicubic2dGetWorkspaceSize": (_I32, [_P, _P, _B, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleBicubic2d": _PHASE2,
    "aclnnUpsampleBicubic2dBackwardGetWorkspaceSize": (_I32, [_P, _P, _P, _B, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleBicubic2dBackward": _PHASE2,
    "aclnnUpsampleNearest3dGetWorkspaceSize": (_I32, [_P, _P, _D, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleNearest3d": _PHASE2,
    "aclnnUpsampleNearestExact3dGetWorkspaceSize": (_I32, [_P, _P, _D, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleNearestExact3d": _PHASE2,
    "aclnnUpsampleNearest3dBackwardGetWorkspaceSize": (_I32, [_P, _P, _P, _D, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleNearest3dBackward": _PHASE2,
    "aclnnUpsampleNearestExact3dBackwardGetWorkspaceSize": (_I32, [_P, _P, _P, _D, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleNearestExact3dBackward": _PHASE2,
    "aclnnUpsampleTrilinear3dGetWorkspaceSize": (_I32, [_P, _P, _B, _D, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleTrilinear3d": _PHASE2,
    "aclnnUpsampleTrilinear3dBackwardGetWorkspaceSize": (_I32, [_P, _P, _P, _B, _D, _D, _D, _P, _PU64, _PP]),
    "aclnnUpsampleTrilinear3dBackward": _PHASE2,
    "aclnnGridSampler3DGetWorkspaceSize": (_I32, [_P, _P, _I64, _I64, _B, _P, _PU64, _PP]),
    "aclnnGridSampler3D": _PHASE2,
    "aclnnGridSampler3DBackwardGetWorkspaceSize": (_I32, [_P, _P, _P, _I64, _I64, _B, _P, _P, _P, _PU64, _PP]),
    "aclnnGridSampler3DBackward": _PHASE2,
    "aclnnResizeGetWorkspaceSize": (_I32, [_P, _P, ctypes.c_char_p, _P, _PU64, _PP]),
    "aclnnResize": _PHASE2,
    "aclnnGridSampler2DGetWorkspaceSize": (_I32, [_P, _P, _I64, _I64, _B, _P, _PU64, _PP]),
    "aclnnGridSampler2D": _PHASE2,
    "aclnnGridSampler2DBackwardGetWorkspaceSize": (_I32, [_P, _P, _P, _I64, _I64, _B, _P, _P, _P, _PU64, _PP]),
    "aclnnGridSampler2DBackward": _PHASE2,
}

_lib = None


def lib():
    """Load the shared library (once). Raises OSError if it has not been built: there is no other code path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OSError(f"{LIB_PATH} not found: build it with __graft_entry__.build() or `make -C {CSRC_DIR}`")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


from .aclnn import *  # noqa: E402,F401,F403
