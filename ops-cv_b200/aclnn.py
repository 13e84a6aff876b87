"""Two-phase aclnn calls over torch CUDA tensors. torch supplies device memory and the current stream only."""
import ctypes

import torch

from . import (ACL_BF16, ACL_DOUBLE, ACL_FLOAT, ACL_FLOAT16, ACL_FORMAT_NCDHW, ACL_FORMAT_NCHW, ACL_FORMAT_NCL, ACL_FORMAT_ND,
               ACL_FORMAT_NDHWC, ACL_FORMAT_NHWC,
               ACL_INT32, ACL_INT64, ACL_OPT_DETERMINISTIC, ACL_UINT8, lib)

__all__ = [
    "AclnnError", "acl_tensor", "int_array", "bool_array", "float_array", "resize", "two_phase", "set_deterministic", "set_backward_algo",
    "launch_count", "reset_launch_count", "async_copy_timeouts", "last_error", "debug_axis_table", "upsample_nearest2d",
    "upsample_nearest2d_backward", "upsample_bilinear2d", "upsample_bilinear2d_no_alloc",
    "upsample_bilinear2d_backward", "upsample_bicubic2d", "upsample_bicubic2d_backward", "upsample_bilinear2d_aa",
    "upsample_bilinear2d_aa_backward", "upsample_nearest_exact2d", "upsample_nearest_exact2d_backward",
    "upsample_nearest_exact1d", "upsample_nearest_exact1d_backward", "upsample_nearest3d",
    "upsample_nearest3d_backward", "upsample_trilinear3d", "upsample_trilinear3d_backward", "grid_sampler3d",
    "grid_sampler3d_backward", "upsample_bicubic2d_aa",
    "upsample_bicubic2d_aa_grad", "grid_sampler2d", "grid_sampler2d_backward", "Workspace",
]

_DTYPES = {torch.float32: ACL_FLOAT, torch.float16: ACL_FLOAT16, torch.bfloat16: ACL_BF16, torch.float64: ACL_DOUBLE,
           torch.uint8: ACL_UINT8, torch.int32: ACL_INT32, torch.int64: ACL_INT64}
_FORMATS = {"NCHW": ACL_FORMAT_NCHW, "NHWC": ACL_FORMAT_NHWC, "ND": ACL_FORMAT_ND, "NCL": ACL_FORMAT_NCL,
            "NCDHW": ACL_FORMAT_NCDHW, "NDHWC": ACL_FORMAT_NDHWC}


class AclnnError(RuntimeError):
    def __init__(self, api, status):
        self.status = status
        super().__init__(f"{api} returned {status}: {last_error()}")


def last_error():
    return lib().aclGetRecentErrMsg().decode()


class _Handle:
    """Owns one acl object and destroys it with the matching destructor."""

    def __init__(self, ptr, destroy, keep=None):
        self.ptr = ptr
        self._destroy = destroy
        self._keep = keep

    def __del__(self):
        if self.ptr:
            self._destroy(self.ptr)
            self.ptr = None


def acl_tensor(t, fmt="NCHW"):
    """aclTensor view of a torch tensor: its sizes, strides (elements) and data pointer; offset 0."""
    dims = (ctypes.c_int64 * t.dim())(*t.shape)
    strides = (ctypes.c_int64 * t.dim())(*t.stride())
    ptr = lib().aclCreateTensor(dims, t.dim(), _DTYPES[t.dtype], strides, 0, _FORMATS[fmt], dims, t.dim(),
                                ctypes.c_void_p(t.data_ptr()))
    if not ptr:
        raise AclnnError("aclCreateTensor", -1)
    return _Handle(ptr, lib().aclDestroyTensor, keep=t)


def int_array(values):
    arr = (ctypes.c_int64 * len(values))(*values)
    return _Handle(lib().aclCreateIntArray(arr, len(values)), lib().aclDestroyIntArray)


def float_array(values):
    arr = (ctypes.c_float * len(values))(*values)
    return _Handle(lib().aclCreateFloatArray(arr, len(values)), lib().aclDestroyFloatArray)


def bool_array(values):
    arr = (ctypes.c_bool * len(values))(*values)
    return _Handle(lib().aclCreateBoolArray(arr, len(values)), lib().aclDestroyBoolArray)


class Workspace:
    """Grow-only device workspace reused across calls (avoids an allocation per call in timed loops)."""

    def __init__(self, device="cuda"):
        self.device = device
        self.buf = None

    def get(self, nbytes):
        if nbytes == 0:
            return None, 0
        if self.buf is None or self.buf.numel() < nbytes:
            self.buf = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        return self.buf, nbytes


def two_phase(name, args, device, workspace=None, stream=None):
    """Run `<name>GetWorkspaceSize(*args, &ws, &executor)` then `<name>(workspace, ws, executor, stream)`."""
    L = lib()
    ws_size = ctypes.c_uint64(0)
    executor = ctypes.c_void_p(None)
    status = getattr(L, name + "GetWorkspaceSize")(*args, ctypes.byref(ws_size), ctypes.byref(executor))
    if status != 0:
        raise AclnnError(name + "GetWorkspaceSize", status)
    buf = None
    if ws_size.value > 0:
        if workspace is not None:
            buf, _ = workspace.get(ws_size.value)
        else:
            buf = torch.empty(ws_size.value, dtype=torch.uint8, device=device)
    if stream is None:
        stream = torch.cuda.current_stream(device).cuda_stream
    status = getattr(L, name)(ctypes.c_void_p(buf.data_ptr() if buf is not None else None), ws_size.value, executor,
                              ctypes.c_void_p(stream))
    if status != 0:
        raise AclnnError(name, status)
    return ws_size.value


def set_deterministic(flag):
    lib().aclrtCtxSetSysParamOpt(ACL_OPT_DETERMINISTIC, 1 if flag else 0)


def set_backward_algo(algo):
    status = lib().opscvSetBackwardAlgo({"gather": 0, "atomic": 1}.get(algo, algo))
    if status != 0:
        raise AclnnError("opscvSetBackwardAlgo", status)


def launch_count():
    return lib().opscvGetLaunchCount()


def reset_launch_count():
    lib().opscvResetLaunchCount()


def async_copy_timeouts():
    """Bounded device-side waits that ran out (0 in a healthy run)."""
    return lib().opscvGetAsyncCopyTimeouts()


def debug_axis_table(kind, in_size, out_size, align=False, user_scale=0.0):
    """Index / weight tables as the device builds them, copied to numpy arrays (see opscvDebugAxisTable)."""
    import numpy as np
    L = lib()
    kinds = {"nearest_fwd": 0, "nearest_bwd": 1, "bilinear": 2, "bicubic_aa": 3, "bilinear_aa": 4}
    k = kinds[kind]
    n = in_size if k == 1 else out_size
    i0 = np.zeros(n, dtype=np.int32)
    i1 = np.zeros(n, dtype=np.int32)
    taps = ctypes.c_int32(0)
    f0 = None
    if k == 2:
        f0 = np.zeros(n, dtype=np.float32)
    if k >= 3:
        status = L.opscvDebugAxisTable(k, in_size, out_size, int(align), user_scale, None, None, None,
                                       ctypes.byref(taps))
        if status != 0:
            raise AclnnError("opscvDebugAxisTable", status)
        f0 = np.zeros((n, taps.value), dtype=np.float32)
    status = L.opscvDebugAxisTable(k, in_size, out_size, int(align), user_scale, i0.ctypes.data, i1.ctypes.data,
                                   f0.ctypes.data if f0 is not None else None, ctypes.byref(taps))
    if status != 0:
        raise AclnnError("opscvDebugAxisTable", status)
    return i0, i1, f0


def _out_shape(x, out_hw, fmt):
    if fmt == "NHWC":
        return (x.shape[0], out_hw[0], out_hw[1], x.shape[3])
    return (x.shape[0], x.shape[1], out_hw[0], out_hw[1])


# ---- operators ------------------------------------------------------------------------------------------------

def upsample_nearest2d(x, out_hw, fmt="NCHW", scales=None, out=None, workspace=None):
    out = torch.empty(_out_shape(x, out_hw, fmt), dtype=x.dtype, device=x.device) if out is None else out
    tx, ty, size = acl_tensor(x, fmt), acl_tensor(out, fmt), int_array(out_hw)
    if scales is None:
        two_phase("aclnnUpsampleNearest2d", [tx.ptr, size.ptr, ty.ptr], x.device, workspace)
    else:
        two_phase("aclnnUpsampleNearest2dV2", [tx.ptr, size.ptr, float(scales[0]), float(scales[1]), ty.ptr],
                  x.device, workspace)
    return out


def upsample_nearest2d_backward(grad_out, out_hw, input_size, fmt="NCHW", scales=(0.0, 0.0), out=None,
                                workspace=None):
    out = torch.empty(tuple(input_size), dtype=grad_out.dtype, device=grad_out.device) if out is None else out
    tg, ty = acl_tensor(grad_out, fmt), acl_tensor(out, fmt)
    osz, isz = int_array(out_hw), int_array(input_size)
    two_phase("aclnnUpsampleNearest2dBackward", [tg.ptr, osz.ptr, isz.ptr, float(scales[0]), float(scales[1]), ty.ptr],
              grad_out.device, workspace)
    return out


def upsample_bilinear2d(x, out_hw, align_corners=False, fmt="NCHW", scales=(0.0, 0.0), out=None, workspace=None):
    out = torch.empty(_out_shape(x, out_hw, fmt), dtype=x.dtype, device=x.device) if out is None else out
    tx, ty, size = acl_tensor(x, fmt), acl_tensor(out, fmt), int_array(out_hw)
    two_phase("aclnnUpsampleBilinear2d", [tx.ptr, size.ptr, bool(align_corners), float(scales[0]), float(scales[1]),
                                          ty.ptr], x.device, workspace)
    return out


def upsample_bilinear2d_no_alloc(x, out_hw, align_corners=False, fmt="NCHW", scales=(0.0, 0.0), out=None):
    """opscvUpsampleBilinear2dNoAlloc: one call, no workspace (tap tables live in the library's device image)."""
    out = torch.empty(_out_shape(x, out_hw, fmt), dtype=x.dtype, device=x.device) if out is None else out
    assert x.is_contiguous() and out.is_contiguous()
    n, c, h, w = (x.shape[0], x.shape[3], x.shape[1], x.shape[2]) if fmt == "NHWC" else tuple(x.shape)
    with torch.cuda.device(x.device):
        status = lib().opscvUpsampleBilinear2dNoAlloc(
            x.data_ptr(), out.data_ptr(), _DTYPES[x.dtype], _FORMATS[fmt], n, c, h, w, int(out_hw[0]), int(out_hw[1]),
            bool(align_corners), float(scales[0]), float(scales[1]), torch.cuda.current_stream(x.device).cuda_stream)
    if status != 0:
        raise AclnnError("opscvUpsampleBilinear2dNoAlloc", status)
    return out


def upsample_bilinear2d_backward(grad_out, out_hw, input_size, align_corners=False, fmt="NCHW", scales=(0.0, 0.0),
                                 out=None, out_dtype=None, v2=False, workspace=None):
    if out is None:
        out = torch.empty(tuple(input_size), dtype=out_dtype or grad_out.dtype, device=grad_out.device)
    tg, ty = acl_tensor(grad_out, fmt), acl_tensor(out, fmt)
    osz, isz = int_array(out_hw), int_array(input_size)
    name = "aclnnUpsampleBilinear2dBackwardV2" if v2 else "aclnnUpsampleBilinear2dBackward"
    two_phase(name, [tg.ptr, osz.ptr, isz.ptr, bool(align_corners), float(scales[0]), float(scales[1]), ty.ptr],
              grad_out.device, workspace)
    return out


def upsample_bicubic2d_aa(x, out_hw, align_corners=False, scales=(0.0, 0.0), out=None, workspace=None):
    out = torch.empty(_out_shape(x, out_hw, "NCHW"), dtype=x.dtype, device=x.device) if out is None else out
    tx, ty, size = acl_tensor(x, "NCHW"), acl_tensor(out, "NCHW"), int_array(out_hw)
    two_phase("aclnnUpsampleBicubic2dAA", [tx.ptr, size.ptr, bool(align_corners), float(scales[0]), float(scales[1]),
                                           ty.ptr], x.device, workspace)
    return out


def upsample_bicubic2d_aa_grad(grad_out, out_hw, input_size, align_corners=False, scales=(0.0, 0.0), out=None,
                               workspace=None):
    out = torch.empty(tuple(input_size), dtype=grad_out.dtype, device=grad_out.device) if out is None else out
    tg, ty = acl_tensor(grad_out, "NCHW"), acl_tensor(out, "NCHW")
    osz, isz = int_array(out_hw), int_array(input_size)
    two_phase("aclnnUpsampleBicubic2dAAGrad", [tg.ptr, osz.ptr, isz.ptr, bool(align_corners), float(scales[0]),
                                               float(scales[1]), ty.ptr], grad_out.device, workspace)
    return out


def upsample_nearest_exact2d(x, out_hw, fmt="NCHW", scales=(0.0, 0.0), out=None, workspace=None):
    out = torch.empty(_out_shape(x, out_hw, fmt), dtype=x.dtype, device=x.device) if out is None else out
    tx, ty, size = acl_tensor(x, fmt), acl_tensor(out, fmt), int_array(out_hw)
    two_phase("aclnnUpsampleNearestExact2d", [tx.ptr, size.ptr, float(scales[0]), float(scales[1]), ty.ptr], x.device,
              workspace)
    return out


def upsample_nearest_exact2d_backward(grad_out, out_hw, input_size, scales=(0.0, 0.0), out=None, workspace=None):
    out = torch.empty(tuple(input_size), dtype=grad_out.dtype, device=grad_out.device) if out is None else out
    tg, ty = acl_tensor(grad_out, "NCHW"), acl_tensor(out, "NCHW")
    osz, isz = int_array(out_hw), int_array(input_size)
    two_phase("aclnnUpsampleNearestExact2dBackward", [tg.ptr, osz.ptr, isz.ptr, float(scales[0]), float(scales[1]),
                                                      ty.ptr], grad_out.device, workspace)
    return out


def upsample_nearest_exact1d(x, out_l, scale=0.0, fmt="NCL", out=None, workspace=None):
    out = torch.empty((x.shape[0], x.shape[1], out_l), dtype=x.dtype, device=x.device) if out is None else out
    tx, ty, size = acl_tensor(x, fmt), acl_tensor(out, fmt), int_array([out_l])
    two_phase("aclnnUpsampleNearestExact1d", [tx.ptr, size.ptr, float(scale), ty.ptr], x.device, workspace)
    return out


def upsample_nearest_exact1d_backward(grad_out, out_l, input_size, scale=0.0, fmt="NCL", out=None, workspace=None):
    out = torch.empty(tuple(input_size), dtype=grad_out.dtype, device=grad_out.device) if out is None else out
    tg, ty = acl_tensor(grad_out, fmt), acl_tensor(out, fmt)
    osz, isz = int_array([out_l]), int_array(input_size)
    two_phase("aclnnUpsampleNearestExact1dBackward", [tg.ptr, osz.ptr, isz.ptr, float(scale), ty.ptr],
              grad_out.device, workspace)
    return out


def upsample_nearest3d(x, out_dhw, fmt="NCDHW", scales=(0.0, 0.0, 0.0), exact=False, out=None, workspace=None):
    if out is None:
        shape = (x.shape[0], *out_dhw, x.shape[4]) if fmt == "NDHWC" else (x.shape[0], x.shape[1], *out_dhw)
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
    tx, ty, size = acl_tensor(x, fmt), acl_tensor(out, fmt), int_array(list(out_dhw))
    name = "aclnnUpsampleNearestExact3d" if exact else "aclnnUpsampleNearest3d"
    two_phase(name, [tx.ptr, size.ptr, float(scales[0]), float(scales[1]), float(scales[2]), ty.ptr], x.device,
              workspace)
    return out


def upsample_nearest3d_backward(grad_out, out_dhw, input_size, fmt="NCDHW", scales=(0.0, 0.0, 0.0), exact=False,
                                out=None, workspace=None):
    out = torch.empty(tuple(input_size), dtype=grad_out.dtype, device=grad_out.device) if out is None else out
    tg, ty = acl_tensor(grad_out, fmt), acl_tensor(out, fmt)
    osz, isz = int_array(list(out_dhw)), int_array(list(input_size))
    name = "aclnnUpsampleNearestExact3dBackward" if exact else "aclnnUpsampleNearest3dBackward"
    two_phase(name, [tg.ptr, osz.ptr, isz.ptr, float(scales[0]), float(scales[1]), float(scales[2]), ty.ptr],
              grad_out.device, workspace)
    return out


def upsample_trilinear3d(x, out_dhw, align_corners=False, fmt="NCDHW", scales=(0.0, 0.0, 0.0), out=None,
                         workspace=None):
    if out is None:
        shape = (x.shape[0], *out_dhw, x.shape[4]) if fmt == "NDHWC" else (x.shape[0], x.shape[1], *out_dhw)
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
    tx, ty, size = acl_tensor(x, fmt), acl_tensor(out, fmt), int_array(list(out_dhw))
    two_phase("aclnnUpsampleTrilinear3d", [tx.ptr, size.ptr, bool(align_corners), float(scales[0]), float(scales[1]),
                                           float(scales[2]), ty.ptr], x.device, workspace)
    return out


def upsample_trilinear3d_backward(grad_out, out_dhw, input_size, align_corners=False, fmt="NCDHW",
                                  scales=(0.0, 0.0, 0.0), out=None, workspace=None):
    """input_size is (N, C, D, H, W) in either format, as in the reference."""
    if out is None:
        n, c, d, h, w = input_size
        shape = (n, d, h, w, c) if fmt == "NDHWC" else (n, c, d, h, w)
        out = torch.empty(shape, dtype=grad_out.dtype, device=grad_out.device)
    tg, ty = acl_tensor(grad_out, fmt), acl_tensor(out, fmt)
    osz, isz = int_array(list(out_dhw)), int_array(list(input_size))
    two_phase("aclnnUpsampleTrilinear3dBackward", [tg.ptr, osz.ptr, isz.ptr, bool(align_corners), float(scales[0]),
                                                   float(scales[1]), float(scales[2]), ty.ptr], grad_out.device,
              workspace)
    return out


def upsample_bilinear2d_aa(x, out_hw, align_corners=False, scales=(0.0, 0.0), out=None, workspace=None):
    out = torch.empty(_out_shape(x, out_hw, "NCHW"), dtype=x.dtype, device=x.device) if out is None else out
    tx, ty, size = acl_tensor(x, "NCHW"), acl_tensor(out, "NCHW"), int_array(out_hw)
    two_phase("aclnnUpsampleBilinear2dAA", [tx.ptr, size.ptr, bool(align_corners), float(scales[0]), float(scales[1]),
                                            ty.ptr], x.device, workspace)
    return out


def upsample_bilinear2d_aa_backward(grad_out, out_hw, input_size, align_corners=False, scales=(0.0, 0.0), out=None,
                                    workspace=None):
    out = torch.empty(tuple(input_size), dtype=grad_out.dtype, device=grad_out.device) if out is None else out
    tg, ty = acl_tensor(grad_out, "NCHW"), acl_tensor(out, "NCHW")
    osz, isz = int_array(out_hw), int_array(input_size)
    two_phase("aclnnUpsampleBilinear2dAABackward", [tg.ptr, osz.ptr, isz.ptr, bool(align_corners), float(scales[0]),
                                                    float(scales[1]), ty.ptr], grad_out.device, workspace)
    return out


def upsample_bicubic2d(x, out_hw, align_corners=False, fmt="NCHW", scales=(0.0, 0.0), out=None, workspace=None):
    out = torch.empty(_out_shape(x, out_hw, fmt), dtype=x.dtype, device=x.device) if out is None else out
    tx, ty, size = acl_tensor(x, fmt), acl_tensor(out, fmt), int_array(out_hw)
    two_phase("aclnnUpsampleBicubic2d", [tx.ptr, size.ptr, bool(align_corners), float(scales[0]), float(scales[1]),
                                         ty.ptr], x.device, workspace)
    return out


def upsample_bicubic2d_backward(grad_out, out_hw, input_size, align_corners=False, fmt="NCHW", scales=(0.0, 0.0),
                                out=None, workspace=None):
    out = torch.empty(tuple(input_size), dtype=grad_out.dtype, device=grad_out.device) if out is None else out
    tg, ty = acl_tensor(grad_out, fmt), acl_tensor(out, fmt)
    osz, isz = int_array(out_hw), int_array(input_size)
    two_phase("aclnnUpsampleBicubic2dBackward", [tg.ptr, osz.ptr, isz.ptr, bool(align_corners), float(scales[0]),
                                                 float(scales[1]), ty.ptr], grad_out.device, workspace)
    return out


def resize(x, scales, mode="bilinear", fmt="NCHW", out=None, workspace=None):
    """aclnnResize: `scales` has one factor per dimension of x; the output extent is floor(extent * factor)."""
    if out is None:
        h_dim, w_dim = (1, 2) if fmt == "NHWC" else (2, 3)
        out_hw = (int(x.shape[h_dim] * float(scales[h_dim])), int(x.shape[w_dim] * float(scales[w_dim])))
        out = torch.empty(_out_shape(x, out_hw, fmt), dtype=x.dtype, device=x.device)
    tx, ty, sc = acl_tensor(x, fmt), acl_tensor(out, fmt), float_array([float(v) for v in scales])
    two_phase("aclnnResize", [tx.ptr, sc.ptr, mode.encode(), ty.ptr], x.device, workspace)
    return out


def grid_sampler2d(x, grid, interpolation=0, padding=0, align_corners=False, out=None, workspace=None):
    if out is None:
        out = torch.empty((x.shape[0], x.shape[1], grid.shape[1], grid.shape[2]), dtype=x.dtype, device=x.device)
    tx, tg, ty = acl_tensor(x, "NCHW"), acl_tensor(grid, "ND"), acl_tensor(out, "NCHW")
    two_phase("aclnnGridSampler2D", [tx.ptr, tg.ptr, int(interpolation), int(padding), bool(align_corners), ty.ptr],
              x.device, workspace)
    return out


def grid_sampler2d_backward(grad_out, x, grid, interpolation=0, padding=0, align_corners=False, mask=(True, True),
                            input_grad=None, grid_grad=None, workspace=None):
    input_grad = torch.empty_like(x) if input_grad is None else input_grad
    grid_grad = torch.empty_like(grid) if grid_grad is None else grid_grad
    tgo, tx, tg = acl_tensor(grad_out, "NCHW"), acl_tensor(x, "NCHW"), acl_tensor(grid, "ND")
    tgi, tgg, m = acl_tensor(input_grad, "NCHW"), acl_tensor(grid_grad, "ND"), bool_array(list(mask))
    two_phase("aclnnGridSampler2DBackward", [tgo.ptr, tx.ptr, tg.ptr, int(interpolation), int(padding),
                                             bool(align_corners), m.ptr, tgi.ptr, tgg.ptr], x.device, workspace)
    return input_grad, grid_grad


def grid_sampler3d(x, grid, interpolation=0, padding=0, align_corners=False, fmt="NCDHW", out=None, workspace=None):
    if out is None:
        n, do, ho, wo = grid.shape[0], grid.shape[1], grid.shape[2], grid.shape[3]
        shape = (n, do, ho, wo, x.shape[4]) if fmt == "NDHWC" else (n, x.shape[1], do, ho, wo)
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
    tx, tg, ty = acl_tensor(x, fmt), acl_tensor(grid, "ND"), acl_tensor(out, fmt)
    two_phase("aclnnGridSampler3D", [tx.ptr, tg.ptr, int(interpolation), int(padding), bool(align_corners), ty.ptr],
              x.device, workspace)
    return out


def grid_sampler3d_backward(grad_out, x, grid, interpolation=0, padding=0, align_corners=False, mask=(True, True),
                            fmt="NCDHW", input_grad=None, grid_grad=None, workspace=None):
    input_grad = torch.empty_like(x) if input_grad is None else input_grad
    grid_grad = torch.empty_like(grid) if grid_grad is None else grid_grad
    tgo, tx, tg = acl_tensor(grad_out, fmt), acl_tensor(x, fmt), acl_tensor(grid, "ND")
    tgi, tgg, m = acl_tensor(input_grad, fmt), acl_tensor(grid_grad, "ND"), bool_array(list(mask))
    two_phase("aclnnGridSampler3DBackward", [tgo.ptr, tx.ptr, tg.ptr, int(interpolation), int(padding),
                                             bool(align_corners), m.ptr, tgi.ptr, tgg.ptr], x.device, workspace)
    return input_grad, grid_grad
