"""First-phase behaviour of the aclnn entry points, without a GPU: the library loads, exports every symbol the
headers declare, and returns the reference's status codes for invalid arguments. Mirrors the reference's
op_api unit tests, which assert only the GetWorkspaceSize status (e.g.
image/upsample_bilinear2d/tests/ut/op_host/op_api/test_aclnn_upsample_bilinear_2d.cpp:92-110: null self ->
ACLNN_ERR_INNER_NULLPTR; image/grid_sampler2_d_grad/tests/ut/op_host/op_api/
test_aclnn_grid_sampler2d_backward.cpp:86-197: one ACLNN_ERR_PARAM_NULLPTR case per tensor, :391-532 integer
dtypes -> ACLNN_ERR_PARAM_INVALID).

No compute call is made: tensors wrap host memory and only phase one runs.
"""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

OK, NULLPTR, INVALID, INNER_NULL = 0, 161001, 161002, 561103


def phase1(ops, name, *args):
    ws = ctypes.c_uint64(123)
    ex = ctypes.c_void_p(None)
    status = getattr(ops.lib(), name + "GetWorkspaceSize")(*args, ctypes.byref(ws), ctypes.byref(ex))
    if ex.value:
        assert ops.lib().aclDestroyAclOpExecutor(ex) == 0
    return status, ws.value


_KEEP = []  # handles must outlive the calls that receive their raw pointers


def T(ops, shape, dtype=torch.float32, fmt="NCHW"):
    h = ops.acl_tensor(torch.zeros(shape, dtype=dtype), fmt)
    _KEEP.append(h)
    return h


def IA(ops, values):
    h = ops.int_array(values)
    _KEEP.append(h)
    return h


def BA(ops, values):
    h = ops.bool_array(values)
    _KEEP.append(h)
    return h


def test_library_exports_every_declared_symbol(ops):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    declared = set()
    for header in ("aclnn_resample.h", "opscv_acl.h"):
        text = open(os.path.join(root, "include", header)).read()
        declared |= set(re.findall(r"ACLNN_API\s+[\w\s\*]+?\b(\w+)\s*\(", text))
    assert len(declared) >= 36
    handle = ctypes.CDLL(ops.LIB_PATH)
    missing = [s for s in sorted(declared) if not hasattr(handle, s)]
    assert not missing, missing
    assert declared == set(ops.SYMBOLS), declared ^ set(ops.SYMBOLS)
    assert ops.lib().opscvVersion() >= 100


def test_nearest_forward_status(ops):
    x, y, sz = T(ops, (2, 3, 4, 5)), T(ops, (2, 3, 8, 10)), IA(ops, [8, 10])
    assert phase1(ops, "aclnnUpsampleNearest2d", x.ptr, sz.ptr, y.ptr)[0] == OK
    assert phase1(ops, "aclnnUpsampleNearest2d", None, sz.ptr, y.ptr)[0] == NULLPTR
    assert phase1(ops, "aclnnUpsampleNearest2d", x.ptr, None, y.ptr)[0] == NULLPTR
    assert phase1(ops, "aclnnUpsampleNearest2d", x.ptr, sz.ptr, None)[0] == NULLPTR
    assert phase1(ops, "aclnnUpsampleNearest2d", x.ptr, sz.ptr, T(ops, (2, 3, 8, 10), torch.float16).ptr)[0] == INVALID
    assert phase1(ops, "aclnnUpsampleNearest2d", T(ops, (2, 3, 4, 5), torch.int32).ptr, sz.ptr,
                  T(ops, (2, 3, 8, 10), torch.int32).ptr)[0] == INVALID
    assert phase1(ops, "aclnnUpsampleNearest2d", x.ptr, IA(ops, [8]).ptr, y.ptr)[0] == INVALID
    assert phase1(ops, "aclnnUpsampleNearest2d", T(ops, (3, 4, 5)).ptr, sz.ptr, y.ptr)[0] == INVALID
    assert phase1(ops, "aclnnUpsampleNearest2d", x.ptr, IA(ops, [8, 11]).ptr, y.ptr)[0] == INVALID
    assert phase1(ops, "aclnnUpsampleNearest2d", x.ptr, sz.ptr, T(ops, (2, 4, 8, 10)).ptr)[0] == INVALID  # C differs
    assert phase1(ops, "aclnnUpsampleNearest2d", x.ptr, sz.ptr, T(ops, (2, 3, 8, 10), fmt="NHWC").ptr)[0] == INVALID
    assert phase1(ops, "aclnnUpsampleNearest2d", T(ops, (2, 3, 4, 5), fmt="ND").ptr, sz.ptr,
                  T(ops, (2, 3, 8, 10), fmt="ND").ptr)[0] == INVALID
    assert phase1(ops, "aclnnUpsampleNearest2d", T(ops, (2, 3, 0, 5)).ptr, sz.ptr, y.ptr)[0] == INVALID
    # empty batch: success without workspace
    st, ws = phase1(ops, "aclnnUpsampleNearest2d", T(ops, (0, 3, 4, 5)).ptr, sz.ptr, T(ops, (0, 3, 8, 10)).ptr)
    assert (st, ws) == (OK, 0)
    # NHWC
    xn, yn = T(ops, (2, 4, 5, 3), fmt="NHWC"), T(ops, (2, 8, 10, 3), fmt="NHWC")
    assert phase1(ops, "aclnnUpsampleNearest2d", xn.ptr, sz.ptr, yn.ptr)[0] == OK
    # V2 takes float scales
    assert phase1(ops, "aclnnUpsampleNearest2dV2", x.ptr, sz.ptr, ctypes.c_float(2.0), ctypes.c_float(2.0),
                  y.ptr)[0] == OK
    assert phase1(ops, "aclnnUpsampleNearest2dV2", None, sz.ptr, ctypes.c_float(2.0), ctypes.c_float(2.0),
                  y.ptr)[0] == NULLPTR


def test_bilinear_forward_status(ops):
    x, y, sz = T(ops, (1, 3, 64, 64)), T(ops, (1, 3, 128, 128)), IA(ops, [128, 128])
    args = lambda a, s, o, sh=0.0, sw=0.0: (a, s, False, sh, sw, o)  # noqa: E731
    st, ws = phase1(ops, "aclnnUpsampleBilinear2d", *args(x.ptr, sz.ptr, y.ptr))
    assert st == OK and ws > 0 and ws % 256 == 0
    # the reference returns the INNER null-pointer code for a null self / out
    assert phase1(ops, "aclnnUpsampleBilinear2d", *args(None, sz.ptr, y.ptr))[0] == INNER_NULL
    assert phase1(ops, "aclnnUpsampleBilinear2d", *args(x.ptr, sz.ptr, None))[0] == INNER_NULL
    assert phase1(ops, "aclnnUpsampleBilinear2d", *args(x.ptr, None, y.ptr))[0] == INVALID
    assert phase1(ops, "aclnnUpsampleBilinear2d", *args(x.ptr, IA(ops, [128]).ptr, y.ptr))[0] == INVALID
    assert phase1(ops, "aclnnUpsampleBilinear2d", *args(x.ptr, IA(ops, [128, 64]).ptr, y.ptr))[0] == INVALID
    assert phase1(ops, "aclnnUpsampleBilinear2d", *args(x.ptr, sz.ptr, y.ptr, -1.0, 2.0))[0] == INVALID
    assert phase1(ops, "aclnnUpsampleBilinear2d", *args(x.ptr, sz.ptr, T(ops, (1, 3, 128, 128), torch.bfloat16).ptr))[0] == INVALID
    assert phase1(ops, "aclnnUpsampleBilinear2d", *args(T(ops, (1, 3, 64, 64), torch.float64).ptr, sz.ptr,
                                                        T(ops, (1, 3, 128, 128), torch.float64).ptr))[0] == INVALID
    assert phase1(ops, "aclnnUpsampleBilinear2d", *args(x.ptr, sz.ptr, T(ops, (2, 3, 128, 128)).ptr))[0] == INVALID
    assert phase1(ops, "aclnnUpsampleBilinear2d", *args(T(ops, (3, 64, 64)).ptr, sz.ptr, y.ptr))[0] == INVALID
    assert phase1(ops, "aclnnUpsampleBilinear2d", *args(x.ptr, sz.ptr, T(ops, (1, 128, 128, 3), fmt="NHWC").ptr))[0] == INVALID
    assert "aclnnUpsampleBilinear2d" in ops.last_error()
    # same size: copy plan, no workspace for contiguous tensors
    st, ws = phase1(ops, "aclnnUpsampleBilinear2d", *args(x.ptr, IA(ops, [64, 64]).ptr, T(ops, (1, 3, 64, 64)).ptr))
    assert (st, ws) == (OK, 0)
    # a strided output needs staging space on top of the tables
    big = torch.zeros((1, 3, 128, 256))
    yv = ops.acl_tensor(big[:, :, :, ::2], "NCHW")
    _KEEP.append(yv)
    st2, ws2 = phase1(ops, "aclnnUpsampleBilinear2d", *args(x.ptr, sz.ptr, yv.ptr))
    assert st2 == OK and ws2 >= ws + 3 * 128 * 128 * 4


def test_backward_status(ops):
    g, out = T(ops, (2, 3, 8, 10)), T(ops, (2, 3, 4, 5))
    osz, isz = IA(ops, [8, 10]), IA(ops, [2, 3, 4, 5])
    for name, extra in (("aclnnUpsampleNearest2dBackward", ()), ("aclnnUpsampleBilinear2dBackward", (False,)),
                        ("aclnnUpsampleBilinear2dBackwardV2", (True,)), ("aclnnUpsampleBicubic2dAAGrad", (False,))):
        def call(gp, op, ip, outp, sh=0.0, sw=0.0):
            return phase1(ops, name, gp, op, ip, *extra, sh, sw, outp)[0]
        assert call(g.ptr, osz.ptr, isz.ptr, out.ptr) == OK, name
        assert call(None, osz.ptr, isz.ptr, out.ptr) == NULLPTR, name
        assert call(g.ptr, None, isz.ptr, out.ptr) == NULLPTR, name
        assert call(g.ptr, osz.ptr, None, out.ptr) == NULLPTR, name
        assert call(g.ptr, osz.ptr, isz.ptr, None) == NULLPTR, name
        assert call(g.ptr, IA(ops, [8]).ptr, isz.ptr, out.ptr) == INVALID, name
        assert call(g.ptr, osz.ptr, IA(ops, [2, 3, 4]).ptr, out.ptr) == INVALID, name
        assert call(g.ptr, IA(ops, [8, 11]).ptr, isz.ptr, out.ptr) == INVALID, name
        if name != "aclnnUpsampleBilinear2dBackward":  # that one lets fp32 grads produce any supported dtype
            assert call(g.ptr, osz.ptr, isz.ptr, T(ops, (2, 3, 4, 5), torch.float16).ptr) == INVALID, name
        assert call(T(ops, (2, 3, 8, 10), torch.int32).ptr, osz.ptr, isz.ptr, T(ops, (2, 3, 4, 5), torch.int32).ptr) == INVALID, name
        assert call(g.ptr, osz.ptr, IA(ops, [2, 3, 0, 5]).ptr, out.ptr) == INVALID, name
    # bilinear backward: fp32 grads may produce a 16-bit gradient (resize_bilinear_v2_grad dtype rule)
    assert phase1(ops, "aclnnUpsampleBilinear2dBackward", g.ptr, osz.ptr, isz.ptr, False, 0.0, 0.0,
                  T(ops, (2, 3, 4, 5), torch.bfloat16).ptr)[0] == OK
    assert phase1(ops, "aclnnUpsampleBilinear2dBackward", T(ops, (2, 3, 8, 10), torch.float16).ptr, osz.ptr, isz.ptr,
                  False, 0.0, 0.0, T(ops, (2, 3, 4, 5), torch.float32).ptr)[0] == INVALID
    # bicubic AA: NCHW / ND only, negative scales rejected
    assert phase1(ops, "aclnnUpsampleBicubic2dAAGrad", T(ops, (2, 8, 10, 3), fmt="NHWC").ptr, osz.ptr,
                  IA(ops, [2, 4, 5, 3]).ptr, False, 0.0, 0.0, T(ops, (2, 4, 5, 3), fmt="NHWC").ptr)[0] == INVALID
    assert phase1(ops, "aclnnUpsampleBicubic2dAAGrad", g.ptr, osz.ptr, isz.ptr, False, -1.0, 0.0, out.ptr)[0] == INVALID


def test_bicubic_aa_forward_status(ops):
    x, y, sz = T(ops, (2, 3, 32, 32)), T(ops, (2, 3, 7, 9)), IA(ops, [7, 9])
    st, ws = phase1(ops, "aclnnUpsampleBicubic2dAA", x.ptr, sz.ptr, False, 0.0, 0.0, y.ptr)
    assert st == OK and ws > 0
    assert phase1(ops, "aclnnUpsampleBicubic2dAA", None, sz.ptr, False, 0.0, 0.0, y.ptr)[0] == NULLPTR
    assert phase1(ops, "aclnnUpsampleBicubic2dAA", x.ptr, None, False, 0.0, 0.0, y.ptr)[0] == NULLPTR
    assert phase1(ops, "aclnnUpsampleBicubic2dAA", x.ptr, sz.ptr, False, 0.0, 0.0, None)[0] == NULLPTR
    assert phase1(ops, "aclnnUpsampleBicubic2dAA", x.ptr, IA(ops, [7, 9, 1]).ptr, False, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, "aclnnUpsampleBicubic2dAA", x.ptr, IA(ops, [7, 8]).ptr, False, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, "aclnnUpsampleBicubic2dAA", x.ptr, IA(ops, [0, 9]).ptr, False, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, "aclnnUpsampleBicubic2dAA", x.ptr, sz.ptr, False, 0.0, 0.0, T(ops, (2, 3, 7, 9), torch.float16).ptr)[0] == INVALID
    assert phase1(ops, "aclnnUpsampleBicubic2dAA", T(ops, (2, 32, 32, 3), fmt="NHWC").ptr, sz.ptr, False, 0.0, 0.0,
                  T(ops, (2, 7, 9, 3), fmt="NHWC").ptr)[0] == INVALID
    assert phase1(ops, "aclnnUpsampleBicubic2dAA", T(ops, (2, 3, 32, 32), fmt="ND").ptr, sz.ptr, False, 0.0, 0.0,
                  T(ops, (2, 3, 7, 9), fmt="ND").ptr)[0] == OK


def test_nearest_exact_status(ops):
    api = "aclnnUpsampleNearestExact2d"
    x, y, sz = T(ops, (2, 3, 8, 8)), T(ops, (2, 3, 16, 12)), IA(ops, [16, 12])
    st, ws = phase1(ops, api, x.ptr, sz.ptr, 0.0, 0.0, y.ptr)
    assert st == OK and ws > 0
    assert phase1(ops, api, None, sz.ptr, 0.0, 0.0, y.ptr)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, None, 0.0, 0.0, y.ptr)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, sz.ptr, 0.0, 0.0, None)[0] == NULLPTR
    # empty tensors succeed before any other check
    assert phase1(ops, api, T(ops, (0, 3, 8, 8)).ptr, IA(ops, [16]).ptr, 0.0, 0.0, T(ops, (0, 3, 16, 12)).ptr) == (OK, 0)
    assert phase1(ops, api, T(ops, (2, 3, 8, 8), torch.int32).ptr, sz.ptr, 0.0, 0.0,
                  T(ops, (2, 3, 16, 12), torch.int32).ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, sz.ptr, 0.0, 0.0, T(ops, (2, 3, 16, 12), torch.float16).ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (3, 8, 8)).ptr, sz.ptr, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, IA(ops, [16, 12, 1]).ptr, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, sz.ptr, 0.0, 0.0, T(ops, (2, 4, 16, 12)).ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, sz.ptr, 0.0, 0.0, T(ops, (2, 3, 16, 12), fmt="NHWC").ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (2, 8, 8, 3), fmt="NHWC").ptr, sz.ptr, 0.0, 0.0,
                  T(ops, (2, 16, 12, 3), fmt="NHWC").ptr)[0] == OK
    api = "aclnnUpsampleNearestExact2dBackward"
    g, out = T(ops, (2, 3, 16, 12)), T(ops, (2, 3, 8, 8))
    osz, isz = IA(ops, [16, 12]), IA(ops, [2, 3, 8, 8])
    st, ws = phase1(ops, api, g.ptr, osz.ptr, isz.ptr, 0.0, 0.0, out.ptr)
    assert st == OK and ws > 0
    assert phase1(ops, api, None, osz.ptr, isz.ptr, 0.0, 0.0, out.ptr)[0] == NULLPTR
    assert phase1(ops, api, g.ptr, osz.ptr, None, 0.0, 0.0, out.ptr)[0] == NULLPTR
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, 0.0, 0.0, None)[0] == NULLPTR
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, -1.0, 0.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, 100.0, 0.0, out.ptr)[0] == INVALID   # up-scale limit of 50
    assert phase1(ops, api, g.ptr, osz.ptr, IA(ops, [2, 3, 8]).ptr, 0.0, 0.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, 0.0, 0.0, T(ops, (2, 3, 8, 8), torch.float16).ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, 0.0, 0.0, T(ops, (2, 4, 8, 8)).ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (2, 16, 12, 3), fmt="NHWC").ptr, osz.ptr, IA(ops, [2, 8, 8, 3]).ptr, 0.0, 0.0,
                  T(ops, (2, 8, 8, 3), fmt="NHWC").ptr)[0] == INVALID


def test_nearest_exact_1d_status(ops):
    api = "aclnnUpsampleNearestExact1d"
    x, y, sz = T(ops, (2, 3, 8), fmt="NCL"), T(ops, (2, 3, 16), fmt="NCL"), IA(ops, [16])
    assert phase1(ops, api, x.ptr, sz.ptr, 0.0, y.ptr)[0] == OK
    assert phase1(ops, api, None, sz.ptr, 0.0, y.ptr)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, None, 0.0, y.ptr)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, sz.ptr, 0.0, None)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, IA(ops, [16, 1]).ptr, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (2, 3, 1, 8)).ptr, sz.ptr, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (0, 3, 8), fmt="NCL").ptr, sz.ptr, 0.0, T(ops, (0, 3, 16), fmt="NCL").ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, sz.ptr, 0.0, T(ops, (2, 3, 16), torch.float16, fmt="NCL").ptr)[0] == INVALID
    # a format the reference has no branch for ends in its inner-null status
    assert phase1(ops, api, T(ops, (2, 3, 8), fmt="NCHW").ptr, sz.ptr, 0.0, T(ops, (2, 3, 16), fmt="NCHW").ptr)[0] == INNER_NULL
    api = "aclnnUpsampleNearestExact1dBackward"
    g, out = T(ops, (2, 3, 16), fmt="NCL"), T(ops, (2, 3, 8), fmt="NCL")
    osz, isz = IA(ops, [16]), IA(ops, [2, 3, 8])
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, 0.0, out.ptr)[0] == OK
    assert phase1(ops, api, None, osz.ptr, isz.ptr, 0.0, out.ptr)[0] == NULLPTR
    assert phase1(ops, api, g.ptr, osz.ptr, None, 0.0, out.ptr)[0] == NULLPTR
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, 0.0, None)[0] == NULLPTR
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, -2.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, 80.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, osz.ptr, IA(ops, [2, 3, 1, 8]).ptr, 0.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, IA(ops, [16, 1]).ptr, isz.ptr, 0.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, 0.0, T(ops, (2, 4, 8), fmt="NCL").ptr)[0] == INVALID


def FA(ops, values):
    h = ops.float_array(values)
    _KEEP.append(h)
    return h


def test_resize_status(ops):
    api = "aclnnResize"
    x, y, sc = T(ops, (2, 3, 8, 8)), T(ops, (2, 3, 16, 12)), FA(ops, [1.0, 1.0, 2.0, 1.5])
    for mode in (b"nearest", b"bilinear", b"nearest-anything"):
        assert phase1(ops, api, x.ptr, sc.ptr, mode, y.ptr)[0] == OK
    assert phase1(ops, api, None, sc.ptr, b"nearest", y.ptr)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, None, b"nearest", y.ptr)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, sc.ptr, None, y.ptr)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, sc.ptr, b"nearest", None)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, sc.ptr, b"bicubic", y.ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, FA(ops, [2.0, 1.5]).ptr, b"nearest", y.ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, FA(ops, [1.0, 1.0, 2.0, 2.0]).ptr, b"nearest", y.ptr)[0] == INVALID   # width 16 != 12
    assert phase1(ops, api, x.ptr, sc.ptr, b"nearest", T(ops, (2, 4, 16, 12)).ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, sc.ptr, b"nearest", T(ops, (2, 3, 16, 12), torch.float16).ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (2, 3, 8, 8), fmt="ND").ptr, sc.ptr, b"nearest", T(ops, (2, 3, 16, 12), fmt="ND").ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (2, 8, 8, 3), fmt="NHWC").ptr, FA(ops, [1.0, 2.0, 1.5, 1.0]).ptr, b"bilinear",
                  T(ops, (2, 16, 12, 3), fmt="NHWC").ptr)[0] == OK
    n = ctypes.c_uint64(0)
    assert ops.lib().aclGetFloatArraySize(sc.ptr, ctypes.byref(n)) == 0 and n.value == 4
    assert ops.lib().aclGetFloatArraySize(None, ctypes.byref(n)) != 0


def test_nearest3d_status(ops):
    for api in ("aclnnUpsampleNearest3d", "aclnnUpsampleNearestExact3d"):
        x, y, sz = T(ops, (2, 3, 4, 8, 8), fmt="NCDHW"), T(ops, (2, 3, 8, 16, 12), fmt="NCDHW"), IA(ops, [8, 16, 12])
        assert phase1(ops, api, x.ptr, sz.ptr, 0.0, 0.0, 0.0, y.ptr)[0] == OK
        assert phase1(ops, api, None, sz.ptr, 0.0, 0.0, 0.0, y.ptr)[0] == NULLPTR
        assert phase1(ops, api, x.ptr, None, 0.0, 0.0, 0.0, y.ptr)[0] == NULLPTR
        assert phase1(ops, api, x.ptr, sz.ptr, 0.0, 0.0, 0.0, None)[0] == NULLPTR
        assert phase1(ops, api, x.ptr, IA(ops, [8, 16]).ptr, 0.0, 0.0, 0.0, y.ptr)[0] == INVALID
        assert phase1(ops, api, x.ptr, IA(ops, [8, 16, 13]).ptr, 0.0, 0.0, 0.0, y.ptr)[0] == INVALID
        assert phase1(ops, api, T(ops, (2, 3, 8, 8)).ptr, sz.ptr, 0.0, 0.0, 0.0, y.ptr)[0] == INVALID
        assert phase1(ops, api, x.ptr, sz.ptr, 0.0, 0.0, 0.0, T(ops, (2, 3, 8, 16, 12), torch.float16, fmt="NCDHW").ptr)[0] == INVALID
        assert phase1(ops, api, T(ops, (2, 0, 4, 8, 8), fmt="NCDHW").ptr, sz.ptr, 0.0, 0.0, 0.0, y.ptr)[0] == INVALID
        assert phase1(ops, api, T(ops, (0, 3, 4, 8, 8), fmt="NCDHW").ptr, sz.ptr, 0.0, 0.0, 0.0,
                      T(ops, (0, 3, 8, 16, 12), fmt="NCDHW").ptr) == (OK, 0)
        assert phase1(ops, api, T(ops, (2, 4, 8, 8, 3), fmt="NDHWC").ptr, sz.ptr, 0.0, 0.0, 0.0,
                      T(ops, (2, 8, 16, 12, 3), fmt="NDHWC").ptr)[0] == OK
    # the exact variant checks positive scales against the sizes
    x, y, sz = T(ops, (2, 3, 4, 8, 8), fmt="NCDHW"), T(ops, (2, 3, 8, 16, 12), fmt="NCDHW"), IA(ops, [8, 16, 12])
    assert phase1(ops, "aclnnUpsampleNearestExact3d", x.ptr, sz.ptr, 2.0, 2.0, 1.5, y.ptr)[0] == OK
    assert phase1(ops, "aclnnUpsampleNearestExact3d", x.ptr, sz.ptr, 2.0, 2.0, 2.0, y.ptr)[0] == INVALID
    for api in ("aclnnUpsampleNearest3dBackward", "aclnnUpsampleNearestExact3dBackward"):
        g, out = T(ops, (2, 3, 8, 16, 12), fmt="NCDHW"), T(ops, (2, 3, 4, 8, 8), fmt="NCDHW")
        osz, isz = IA(ops, [8, 16, 12]), IA(ops, [2, 3, 4, 8, 8])
        assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, 0.0, 0.0, 0.0, out.ptr)[0] == OK
        assert phase1(ops, api, None, osz.ptr, isz.ptr, 0.0, 0.0, 0.0, out.ptr)[0] == NULLPTR
        assert phase1(ops, api, g.ptr, None, isz.ptr, 0.0, 0.0, 0.0, out.ptr)[0] == NULLPTR
        assert phase1(ops, api, g.ptr, osz.ptr, None, 0.0, 0.0, 0.0, out.ptr)[0] == NULLPTR
        assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, 0.0, 0.0, 0.0, None)[0] == NULLPTR
        assert phase1(ops, api, g.ptr, osz.ptr, IA(ops, [2, 3, 4, 8]).ptr, 0.0, 0.0, 0.0, out.ptr)[0] == INVALID
        assert phase1(ops, api, g.ptr, IA(ops, [8, 16, 13]).ptr, isz.ptr, 0.0, 0.0, 0.0, out.ptr)[0] == INVALID
        assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, 0.0, 0.0, 0.0, T(ops, (2, 3, 4, 8, 9), fmt="NCDHW").ptr)[0] == INVALID
    assert phase1(ops, "aclnnUpsampleNearestExact3dBackward", g.ptr, osz.ptr, isz.ptr, -1.0, 0.0, 0.0, out.ptr)[0] == INVALID
    assert phase1(ops, "aclnnUpsampleNearestExact3dBackward", g.ptr, osz.ptr, isz.ptr, 90.0, 0.0, 0.0, out.ptr)[0] == INVALID


def test_grid_sampler3d_status(ops):
    api = "aclnnGridSampler3D"
    x, grid, out = T(ops, (2, 3, 4, 5, 6), fmt="NCDHW"), T(ops, (2, 3, 4, 5, 3), fmt="ND"), T(ops, (2, 3, 3, 4, 5), fmt="NCDHW")
    assert phase1(ops, api, x.ptr, grid.ptr, 0, 0, False, out.ptr)[0] == OK
    assert phase1(ops, api, x.ptr, grid.ptr, 1, 2, True, out.ptr)[0] == OK
    assert phase1(ops, api, None, grid.ptr, 0, 0, False, out.ptr)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, None, 0, 0, False, out.ptr)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, grid.ptr, 0, 0, False, None)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, grid.ptr, 2, 0, False, out.ptr)[0] == INVALID     # no bicubic in 3-D
    assert phase1(ops, api, x.ptr, grid.ptr, 0, 3, False, out.ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, T(ops, (2, 3, 4, 5, 2), fmt="ND").ptr, 0, 0, False, out.ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, T(ops, (2, 3, 4, 5, 3), torch.float16, fmt="ND").ptr, 0, 0, False, out.ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, grid.ptr, 0, 0, False, T(ops, (2, 4, 3, 4, 5), fmt="NCDHW").ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (2, 3, 5, 6), fmt="ND").ptr, grid.ptr, 0, 0, False, out.ptr)[0] == INVALID
    api = "aclnnGridSampler3DBackward"
    go, gi, gg, mask = T(ops, (2, 3, 3, 4, 5), fmt="NCDHW"), T(ops, (2, 3, 4, 5, 6), fmt="NCDHW"), T(ops, (2, 3, 4, 5, 3), fmt="ND"), BA(ops, [True, True])
    assert phase1(ops, api, go.ptr, x.ptr, grid.ptr, 0, 0, False, mask.ptr, gi.ptr, gg.ptr)[0] == OK
    assert phase1(ops, api, go.ptr, x.ptr, grid.ptr, 0, 0, False, None, gi.ptr, gg.ptr)[0] == NULLPTR
    assert phase1(ops, api, None, x.ptr, grid.ptr, 0, 0, False, mask.ptr, gi.ptr, gg.ptr)[0] == NULLPTR
    assert phase1(ops, api, go.ptr, x.ptr, grid.ptr, 0, 0, False, mask.ptr, None, gg.ptr)[0] == NULLPTR
    assert phase1(ops, api, go.ptr, x.ptr, grid.ptr, 0, 0, False, BA(ops, [True]).ptr, gi.ptr, gg.ptr)[0] == INVALID
    assert phase1(ops, api, go.ptr, x.ptr, grid.ptr, 2, 0, False, mask.ptr, gi.ptr, gg.ptr)[0] == INVALID
    assert phase1(ops, api, go.ptr, x.ptr, grid.ptr, 0, 0, False, mask.ptr, T(ops, (2, 3, 4, 5, 7), fmt="NCDHW").ptr, gg.ptr)[0] == INVALID
    assert phase1(ops, api, go.ptr, x.ptr, grid.ptr, 0, 0, False, BA(ops, [False, False]).ptr, gi.ptr, gg.ptr) == (OK, 0)


def test_bilinear_aa_status(ops):
    """aclnnUpsampleBilinear2dAA / ...Backward: the checks of the bicubic-AA pair (NCHW or ND only, one dtype, 4-D,
    sizes > 0) plus negative scales in the forward."""
    api = "aclnnUpsampleBilinear2dAA"
    x, y, sz = T(ops, (2, 3, 32, 32)), T(ops, (2, 3, 7, 9)), IA(ops, [7, 9])
    st, ws = phase1(ops, api, x.ptr, sz.ptr, False, 0.0, 0.0, y.ptr)
    assert st == OK and ws > 0
    assert phase1(ops, api, None, sz.ptr, False, 0.0, 0.0, y.ptr)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, None, False, 0.0, 0.0, y.ptr)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, sz.ptr, False, 0.0, 0.0, None)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, sz.ptr, False, -1.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, IA(ops, [7, 8]).ptr, False, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, IA(ops, [0, 9]).ptr, False, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, sz.ptr, False, 0.0, 0.0, T(ops, (2, 3, 7, 9), torch.bfloat16).ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (2, 3, 32, 32), torch.int32).ptr, sz.ptr, False, 0.0, 0.0,
                  T(ops, (2, 3, 7, 9), torch.int32).ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (2, 32, 32, 3), fmt="NHWC").ptr, sz.ptr, False, 0.0, 0.0,
                  T(ops, (2, 7, 9, 3), fmt="NHWC").ptr)[0] == INVALID
    api = "aclnnUpsampleBilinear2dAABackward"
    g, out = T(ops, (2, 3, 7, 9)), T(ops, (2, 3, 32, 32))
    osz, isz = IA(ops, [7, 9]), IA(ops, [2, 3, 32, 32])
    st, ws = phase1(ops, api, g.ptr, osz.ptr, isz.ptr, False, 0.0, 0.0, out.ptr)
    assert st == OK and ws > 0
    assert phase1(ops, api, None, osz.ptr, isz.ptr, False, 0.0, 0.0, out.ptr)[0] == NULLPTR
    assert phase1(ops, api, g.ptr, osz.ptr, None, False, 0.0, 0.0, out.ptr)[0] == NULLPTR
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, False, 0.0, 0.0, None)[0] == NULLPTR
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, False, 0.0, -2.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, osz.ptr, IA(ops, [2, 3, 32]).ptr, False, 0.0, 0.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, IA(ops, [7, 8]).ptr, isz.ptr, False, 0.0, 0.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, False, 0.0, 0.0, T(ops, (2, 3, 32, 32), torch.float16).ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, False, 0.0, 0.0, T(ops, (2, 4, 32, 32)).ptr)[0] == INVALID


def test_bicubic_forward_status(ops):
    """image/upsample_bicubic2d/tests/ut/op_host/op_api/test_aclnn_upsample_bicubic_2d.cpp:27-310: one null case per
    pointer, float / float16 / bfloat16 succeed, int64 and mixed dtypes are invalid, N = 0 succeeds, C = 0, H = 0,
    an output size of 0, three output sizes and 3-D tensors are invalid."""
    api = "aclnnUpsampleBicubic2d"
    x, y, sz = T(ops, (1, 1, 3, 3)), T(ops, (1, 1, 5, 5)), IA(ops, [5, 5])
    st, ws = phase1(ops, api, x.ptr, sz.ptr, False, 0.0, 0.0, y.ptr)
    assert st == OK and ws == 0
    assert phase1(ops, api, None, sz.ptr, False, 0.0, 0.0, y.ptr)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, None, False, 0.0, 0.0, y.ptr)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, sz.ptr, False, 0.0, 0.0, None)[0] == NULLPTR
    for dt in (torch.float16, torch.bfloat16):
        assert phase1(ops, api, T(ops, (1, 1, 3, 3), dt).ptr, sz.ptr, False, 0.0, 0.0, T(ops, (1, 1, 5, 5), dt).ptr)[0] == OK
    assert phase1(ops, api, T(ops, (1, 1, 3, 3), torch.int64).ptr, sz.ptr, False, 0.0, 0.0,
                  T(ops, (1, 1, 5, 5), torch.int64).ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, sz.ptr, False, 0.0, 0.0, T(ops, (1, 1, 5, 5), torch.float16).ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (0, 1, 3, 3)).ptr, sz.ptr, False, 0.0, 0.0, T(ops, (0, 1, 5, 5)).ptr) == (OK, 0)
    assert phase1(ops, api, T(ops, (1, 0, 3, 3)).ptr, sz.ptr, False, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (1, 1, 0, 3)).ptr, sz.ptr, False, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, IA(ops, [5, 0]).ptr, False, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, IA(ops, [5, 5, 5]).ptr, False, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (1, 3, 3)).ptr, sz.ptr, False, 0.0, 0.0, T(ops, (1, 5, 5)).ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, sz.ptr, False, 0.0, 0.0, T(ops, (1, 1, 5, 6)).ptr)[0] == INVALID
    # NHWC and ND are accepted, a format mismatch is not
    assert phase1(ops, api, T(ops, (1, 3, 3, 2), fmt="NHWC").ptr, sz.ptr, True, 0.0, 0.0,
                  T(ops, (1, 5, 5, 2), fmt="NHWC").ptr)[0] == OK
    assert phase1(ops, api, T(ops, (1, 1, 3, 3), fmt="ND").ptr, sz.ptr, False, 0.0, 0.0,
                  T(ops, (1, 1, 5, 5), fmt="ND").ptr)[0] == OK
    assert phase1(ops, api, x.ptr, sz.ptr, False, 0.0, 0.0, T(ops, (1, 1, 5, 5), fmt="NHWC").ptr)[0] == INVALID


def test_bicubic_backward_status(ops):
    """image/upsample_bicubic2d_grad/tests/ut/op_host/op_api/test_aclnn_upsample_bicubic_2d_backward.cpp: float and
    float16 succeed, every other dtype is invalid, N = 0 succeeds, 2-D / 5-D gradOut, a dtype mismatch and sizes that
    disagree with the tensors are invalid."""
    api = "aclnnUpsampleBicubic2dBackward"
    g, out = T(ops, (1, 1, 2, 2)), T(ops, (1, 1, 3, 3))
    osz, isz = IA(ops, [2, 2]), IA(ops, [1, 1, 3, 3])
    st, ws = phase1(ops, api, g.ptr, osz.ptr, isz.ptr, False, 2.0, 2.0, out.ptr)
    assert st == OK and ws == 0
    for args in ((None, osz.ptr, isz.ptr, out.ptr), (g.ptr, None, isz.ptr, out.ptr), (g.ptr, osz.ptr, None, out.ptr),
                 (g.ptr, osz.ptr, isz.ptr, None)):
        assert phase1(ops, api, args[0], args[1], args[2], False, 2.0, 2.0, args[3])[0] == NULLPTR
    for dt, want in ((torch.float16, OK), (torch.bfloat16, OK), (torch.float64, INVALID), (torch.int32, INVALID),
                     (torch.int64, INVALID), (torch.uint8, INVALID)):
        assert phase1(ops, api, T(ops, (1, 1, 2, 2), dt).ptr, osz.ptr, isz.ptr, False, 2.0, 2.0,
                      T(ops, (1, 1, 3, 3), dt).ptr)[0] == want
    assert phase1(ops, api, T(ops, (0, 1, 2, 2)).ptr, osz.ptr, IA(ops, [0, 1, 3, 3]).ptr, False, 2.0, 2.0,
                  T(ops, (0, 1, 3, 3)).ptr) == (OK, 0)
    assert phase1(ops, api, T(ops, (2, 2)).ptr, osz.ptr, isz.ptr, False, 2.0, 2.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (1, 1, 1, 2, 2)).ptr, osz.ptr, isz.ptr, False, 2.0, 2.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, False, 2.0, 2.0, T(ops, (1, 1, 3, 3), torch.float16).ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, IA(ops, [2, 3]).ptr, isz.ptr, False, 2.0, 2.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, IA(ops, [2]).ptr, isz.ptr, False, 2.0, 2.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, osz.ptr, IA(ops, [1, 1, 3]).ptr, False, 2.0, 2.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, osz.ptr, IA(ops, [1, 1, 3, 4]).ptr, False, 2.0, 2.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, osz.ptr, IA(ops, [1, 1, 0, 3]).ptr, False, 2.0, 2.0, T(ops, (1, 1, 0, 3)).ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (1, 2, 2, 4), fmt="NHWC").ptr, osz.ptr, IA(ops, [1, 3, 3, 4]).ptr, True, 0.0, 0.0,
                  T(ops, (1, 3, 3, 4), fmt="NHWC").ptr)[0] == OK
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, False, 2.0, 2.0, T(ops, (1, 1, 3, 3), fmt="NHWC").ptr)[0] == INVALID


def test_grid_sampler_status(ops):
    x, grid, out = T(ops, (2, 3, 6, 7)), T(ops, (2, 5, 4, 2), fmt="ND"), T(ops, (2, 3, 5, 4))
    call = lambda *a: phase1(ops, "aclnnGridSampler2D", *a)[0]  # noqa: E731
    assert call(x.ptr, grid.ptr, 0, 0, False, out.ptr) == OK
    assert call(None, grid.ptr, 0, 0, False, out.ptr) == NULLPTR
    assert call(x.ptr, None, 0, 0, False, out.ptr) == NULLPTR
    assert call(x.ptr, grid.ptr, 0, 0, False, None) == NULLPTR
    for bad in (-1, 3):
        assert call(x.ptr, grid.ptr, bad, 0, False, out.ptr) == INVALID
        assert call(x.ptr, grid.ptr, 0, bad, False, out.ptr) == INVALID
    assert call(x.ptr, T(ops, (2, 5, 4, 2), torch.float16, "ND").ptr, 0, 0, False, out.ptr) == INVALID
    assert call(x.ptr, grid.ptr, 0, 0, False, T(ops, (2, 3, 5, 4), torch.float16).ptr) == INVALID
    for dt in (torch.uint8, torch.int32, torch.int64, torch.float64):
        assert call(T(ops, (2, 3, 6, 7), dt).ptr, T(ops, (2, 5, 4, 2), dt, "ND").ptr, 0, 0, False,
                    T(ops, (2, 3, 5, 4), dt).ptr) == INVALID
    assert call(x.ptr, T(ops, (3, 5, 4, 2), fmt="ND").ptr, 0, 0, False, out.ptr) == INVALID      # batch
    assert call(x.ptr, grid.ptr, 0, 0, False, T(ops, (2, 4, 5, 4)).ptr) == INVALID                # channels
    assert call(x.ptr, grid.ptr, 0, 0, False, T(ops, (2, 3, 5, 5)).ptr) == INVALID                # H/W
    assert call(x.ptr, T(ops, (2, 5, 4, 3), fmt="ND").ptr, 0, 0, False, out.ptr) == INVALID       # last dim != 2
    assert call(T(ops, (2, 3, 0, 7)).ptr, grid.ptr, 0, 0, False, out.ptr) == INVALID
    assert call(T(ops, (3, 6, 7)).ptr, grid.ptr, 0, 0, False, out.ptr) == INVALID


def test_grid_sampler_backward_status(ops):
    x, grid, go = T(ops, (1, 1, 5, 8)), T(ops, (1, 3, 3, 2), fmt="ND"), T(ops, (1, 1, 3, 3))
    gi, gg, mask = T(ops, (1, 1, 5, 8)), T(ops, (1, 3, 3, 2), fmt="ND"), BA(ops, [True, True])

    def call(go_, x_, grid_, gi_, gg_, mask_=mask.ptr, interp=0, pad=0):
        return phase1(ops, "aclnnGridSampler2DBackward", go_, x_, grid_, interp, pad, False, mask_, gi_, gg_)

    st, ws = call(go.ptr, x.ptr, grid.ptr, gi.ptr, gg.ptr)
    assert st == OK and ws == 0  # fp32, atomic mode: accumulates in place
    for i in range(5):  # one null tensor at a time
        args = [go.ptr, x.ptr, grid.ptr, gi.ptr, gg.ptr]
        args[i] = None
        assert call(*args)[0] == NULLPTR
    assert call(go.ptr, x.ptr, grid.ptr, gi.ptr, gg.ptr, mask_=None) == (OK, 0)          # null mask: no-op
    assert call(go.ptr, x.ptr, grid.ptr, gi.ptr, gg.ptr, mask_=BA(ops, [False, False]).ptr) == (OK, 0)
    assert call(go.ptr, x.ptr, grid.ptr, gi.ptr, gg.ptr, mask_=BA(ops, [True]).ptr)[0] == INVALID
    assert call(go.ptr, x.ptr, grid.ptr, gi.ptr, gg.ptr, interp=3)[0] == INVALID
    # all three interpolation modes are accepted, bicubic included (aclnn_grid_sampler2d_backward.cpp:40-41,92-99)
    for mode in (0, 1, 2):
        assert call(go.ptr, x.ptr, grid.ptr, gi.ptr, gg.ptr, interp=mode)[0] == OK
    assert call(go.ptr, x.ptr, grid.ptr, gi.ptr, gg.ptr, pad=-1)[0] == INVALID
    assert call(go.ptr, x.ptr, grid.ptr, T(ops, (1, 1, 5, 7)).ptr, gg.ptr)[0] == INVALID
    assert call(go.ptr, x.ptr, grid.ptr, gi.ptr, T(ops, (1, 3, 4, 2), fmt="ND").ptr)[0] == INVALID
    assert call(T(ops, (1, 2, 3, 3)).ptr, x.ptr, grid.ptr, gi.ptr, gg.ptr)[0] == INVALID
    for dt in (torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64, torch.bool):
        if dt not in (torch.uint8, torch.int32, torch.int64):
            continue  # the ctypes caller maps only these integer dtypes
        assert call(T(ops, (1, 1, 3, 3), dt).ptr, T(ops, (1, 1, 5, 8), dt).ptr, T(ops, (1, 3, 3, 2), dt, "ND").ptr,
                    T(ops, (1, 1, 5, 8), dt).ptr, T(ops, (1, 3, 3, 2), dt, "ND").ptr)[0] == INVALID
    assert call(T(ops, (1, 1, 3, 3), torch.float16).ptr, x.ptr, grid.ptr, gi.ptr, gg.ptr)[0] == INVALID
    # 16-bit tensors accumulate in an fp32 workspace; deterministic mode needs the segment lists
    h = torch.float16
    st, ws16 = call(T(ops, (1, 1, 3, 3), h).ptr, T(ops, (1, 1, 5, 8), h).ptr, T(ops, (1, 3, 3, 2), h, "ND").ptr,
                    T(ops, (1, 1, 5, 8), h).ptr, T(ops, (1, 3, 3, 2), h, "ND").ptr)
    assert st == OK and ws16 >= 40 * 4
    ops.set_deterministic(True)
    try:
        st, wsdet = call(go.ptr, x.ptr, grid.ptr, gi.ptr, gg.ptr)
    finally:
        ops.set_deterministic(False)
    assert st == OK and wsdet >= 4 * 9 * 8


def test_options_and_executor_lifecycle(ops):
    L = ops.lib()
    v = ctypes.c_int64(-1)
    assert L.aclrtCtxGetSysParamOpt(0, ctypes.byref(v)) == 0 and v.value == 0
    assert L.aclrtCtxSetSysParamOpt(0, 1) == 0
    assert L.aclrtCtxGetSysParamOpt(0, ctypes.byref(v)) == 0 and v.value == 1
    assert L.aclrtCtxSetSysParamOpt(0, 0) == 0
    assert L.aclrtCtxSetSysParamOpt(7, 0) != 0
    assert L.opscvSetBackwardAlgo(1) == 0 and L.opscvGetBackwardAlgo() == 1
    assert L.opscvSetBackwardAlgo(5) == INVALID
    assert L.opscvSetBackwardAlgo(0) == 0
    # executors: destroying twice, or running a destroyed one, is rejected instead of touching freed memory
    x, y, sz = T(ops, (1, 3, 4, 4)), T(ops, (1, 3, 8, 8)), IA(ops, [8, 8])
    ws, ex = ctypes.c_uint64(0), ctypes.c_void_p(None)
    assert L.aclnnUpsampleNearest2dGetWorkspaceSize(x.ptr, sz.ptr, y.ptr, ctypes.byref(ws), ctypes.byref(ex)) == 0
    # second phase validates the workspace before any CUDA call
    assert L.aclnnUpsampleNearest2d(None, ws.value, ex, None) == NULLPTR
    assert L.aclnnUpsampleNearest2d(ctypes.c_void_p(256), ws.value - 1, ex, None) == INVALID
    assert L.aclnnUpsampleNearest2d(ctypes.c_void_p(257), ws.value, ex, None) == INVALID
    assert L.aclnnUpsampleBilinear2d(ctypes.c_void_p(256), ws.value, ex, None) == INVALID  # wrong operator
    assert L.aclDestroyAclOpExecutor(ex) == 0
    assert L.aclDestroyAclOpExecutor(ex) == INVALID
    assert L.aclnnUpsampleNearest2d(ctypes.c_void_p(256), ws.value, ex, None) == INVALID
    assert L.aclnnUpsampleNearest2d(ctypes.c_void_p(256), ws.value, None, None) == NULLPTR
    assert L.aclCreateTensor(None, 4, 0, None, 0, 0, None, 0, None) is None


def test_second_phase_without_a_device_reports_a_runtime_error():
    """Phase 2 with no CUDA device visible: the first launch fails, the call returns ACLNN_ERR_RUNTIME_ERROR (361001)
    with the CUDA error in the message, and the executor is consumed. Run in a child process with
    CUDA_VISIBLE_DEVICES empty, so that it means the same on a machine that has GPUs (nothing can be launched there
    either, whatever the pointers are)."""
    import subprocess
    import sys
    code = (
        "import ctypes, os, sys\n"
        f"sys.path.insert(0, {ROOT!r})\n"
        "import __graft_entry__ as entry\n"
        "ops = entry.load_package(); L = ops.lib()\n"
        "dims = (ctypes.c_int64 * 4)(1, 1, 4, 4); odims = (ctypes.c_int64 * 4)(1, 1, 8, 8)\n"
        "st = (ctypes.c_int64 * 4)(16, 16, 4, 1); ost = (ctypes.c_int64 * 4)(64, 64, 8, 1)\n"
        "x = L.aclCreateTensor(dims, 4, 0, st, 0, 0, dims, 4, ctypes.c_void_p(4096))\n"
        "y = L.aclCreateTensor(odims, 4, 0, ost, 0, 0, odims, 4, ctypes.c_void_p(8192))\n"
        "size = (ctypes.c_int64 * 2)(8, 8); sz = L.aclCreateIntArray(size, 2)\n"
        "ws, ex = ctypes.c_uint64(0), ctypes.c_void_p(None)\n"
        "assert L.aclnnUpsampleBilinear2dGetWorkspaceSize(x, sz, False, 0.0, 0.0, y, ctypes.byref(ws), ctypes.byref(ex)) == 0\n"
        "status = L.aclnnUpsampleBilinear2d(ctypes.c_void_p(1 << 20), ws.value, ex, None)\n"
        "msg = L.aclGetRecentErrMsg().decode()\n"
        "again = L.aclnnUpsampleBilinear2d(ctypes.c_void_p(1 << 20), ws.value, ex, None)\n"
        "print(status, again, msg)\n"
    )
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=120)
    assert out.returncode == 0, out.stderr[-2000:]
    status, again, msg = out.stdout.strip().split(" ", 2)
    assert int(status) == 361001 and "CUDA error" in msg
    assert int(again) == INVALID  # the executor was consumed by the failed call


def test_trilinear3d_status(ops):
    api = "aclnnUpsampleTrilinear3d"
    x, y, sz = T(ops, (2, 3, 4, 8, 8), fmt="NCDHW"), T(ops, (2, 3, 8, 16, 12), fmt="NCDHW"), IA(ops, [8, 16, 12])
    assert phase1(ops, api, x.ptr, sz.ptr, False, 0.0, 0.0, 0.0, y.ptr)[0] == OK
    assert phase1(ops, api, x.ptr, sz.ptr, True, 2.0, 2.0, 1.5, y.ptr)[0] == OK
    assert phase1(ops, api, None, sz.ptr, False, 0.0, 0.0, 0.0, y.ptr)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, None, False, 0.0, 0.0, 0.0, y.ptr)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, sz.ptr, False, 0.0, 0.0, 0.0, None)[0] == NULLPTR
    assert phase1(ops, api, x.ptr, IA(ops, [8, 16]).ptr, False, 0.0, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, IA(ops, [8, 16, 13]).ptr, False, 0.0, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, IA(ops, [8, 0, 12]).ptr, False, 0.0, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (2, 3, 8, 8)).ptr, sz.ptr, False, 0.0, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, x.ptr, sz.ptr, False, 0.0, 0.0, 0.0,
                  T(ops, (2, 3, 8, 16, 12), torch.float16, fmt="NCDHW").ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (2, 3, 4, 8, 8), torch.int32, fmt="NCDHW").ptr, sz.ptr, False, 0.0, 0.0, 0.0,
                  T(ops, (2, 3, 8, 16, 12), torch.int32, fmt="NCDHW").ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (2, 3, 4, 8, 8), fmt="NCHW").ptr, sz.ptr, False, 0.0, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (2, 0, 4, 8, 8), fmt="NCDHW").ptr, sz.ptr, False, 0.0, 0.0, 0.0, y.ptr)[0] == INVALID
    assert phase1(ops, api, T(ops, (0, 3, 4, 8, 8), fmt="NCDHW").ptr, sz.ptr, False, 0.0, 0.0, 0.0,
                  T(ops, (0, 3, 8, 16, 12), fmt="NCDHW").ptr) == (OK, 0)
    assert phase1(ops, api, T(ops, (2, 4, 8, 8, 3), fmt="NDHWC").ptr, sz.ptr, False, 0.0, 0.0, 0.0,
                  T(ops, (2, 8, 16, 12, 3), fmt="NDHWC").ptr)[0] == OK
    api = "aclnnUpsampleTrilinear3dBackward"
    g, out = T(ops, (2, 3, 8, 16, 12), fmt="NCDHW"), T(ops, (2, 3, 4, 8, 8), fmt="NCDHW")
    osz, isz = IA(ops, [8, 16, 12]), IA(ops, [2, 3, 4, 8, 8])
    st, ws = phase1(ops, api, g.ptr, osz.ptr, isz.ptr, False, 0.0, 0.0, 0.0, out.ptr)
    assert st == OK and ws > 0  # the per-axis weight lists live in the workspace
    assert phase1(ops, api, None, osz.ptr, isz.ptr, False, 0.0, 0.0, 0.0, out.ptr)[0] == NULLPTR
    assert phase1(ops, api, g.ptr, None, isz.ptr, False, 0.0, 0.0, 0.0, out.ptr)[0] == NULLPTR
    assert phase1(ops, api, g.ptr, osz.ptr, None, False, 0.0, 0.0, 0.0, out.ptr)[0] == NULLPTR
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, False, 0.0, 0.0, 0.0, None)[0] == NULLPTR
    assert phase1(ops, api, g.ptr, osz.ptr, IA(ops, [2, 3, 4, 8]).ptr, False, 0.0, 0.0, 0.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, IA(ops, [8, 16, 13]).ptr, isz.ptr, False, 0.0, 0.0, 0.0, out.ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, False, 0.0, 0.0, 0.0,
                  T(ops, (2, 3, 4, 8, 9), fmt="NCDHW").ptr)[0] == INVALID
    assert phase1(ops, api, g.ptr, osz.ptr, isz.ptr, False, 0.0, 0.0, 0.0,
                  T(ops, (2, 3, 4, 8, 8), torch.float16, fmt="NCDHW").ptr)[0] == INVALID
    # input_size stays (N, C, D, H, W) for NDHWC tensors
    assert phase1(ops, api, T(ops, (2, 8, 16, 12, 3), fmt="NDHWC").ptr, osz.ptr, isz.ptr, True, 0.0, 0.0, 0.0,
                  T(ops, (2, 4, 8, 8, 3), fmt="NDHWC").ptr)[0] == OK
    assert phase1(ops, api, T(ops, (0, 3, 8, 16, 12), fmt="NCDHW").ptr, osz.ptr, IA(ops, [0, 3, 4, 8, 8]).ptr, False,
                  0.0, 0.0, 0.0, T(ops, (0, 3, 4, 8, 8), fmt="NCDHW").ptr) == (OK, 0)
