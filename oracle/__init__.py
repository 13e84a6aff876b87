"""ctypes binding of the CPU oracle (oracle/resample_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline
legs as the checker / the timed CPU baseline. The product library never loads it.

Every function takes and returns fp32 numpy arrays. For 16-bit storage dtypes the caller up-casts the
inputs (exact) and rounds the fp32 result once, which is the "compute in fp32, cast at the end" rule of
the reference kernels.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

NCHW, NHWC = 0, 1
BILINEAR, NEAREST, BICUBIC = 0, 1, 2
ZEROS, BORDER, REFLECTION = 0, 1, 2


def build(force=False):
    """Compile liboracle.so with the Makefile beside this file (gcc only, a few seconds)."""
    src = os.path.join(_HERE, "resample_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def num_threads():
    """OpenMP threads the oracle's loops use."""
    return int(lib().oracle_num_threads())


def set_num_threads(n):
    lib().oracle_set_num_threads(int(n))


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(ctypes.c_void_p)


def _i32(n):
    a = np.zeros(n, dtype=np.int32)
    return a, a.ctypes.data_as(ctypes.c_void_p)


def _dims(shape, fmt):
    if fmt == NCHW:
        n, c, h, w = shape
    else:
        n, h, w, c = shape
    return n, c, h, w


def _shape(n, c, h, w, fmt):
    return (n, c, h, w) if fmt == NCHW else (n, h, w, c)


I64, F32, I32, F64 = ctypes.c_int64, ctypes.c_float, ctypes.c_int, ctypes.c_double


# ---- tables (index / weight computations, compared bit for bit) -----------------------------------------

def nearest_src_index(in_size, out_size, user_scale=0.0):
    idx, p = _i32(out_size)
    lib().orc_nearest_src_index(I64(in_size), I64(out_size), F32(user_scale), p)
    return idx


def nearest_bwd_ranges(in_size, out_size, user_scale=0.0):
    s, ps = _i32(in_size)
    e, pe = _i32(in_size)
    lib().orc_nearest_bwd_ranges(I64(in_size), I64(out_size), F32(user_scale), ps, pe)
    return s, e


def bilinear_table(in_size, out_size, align, user_scale=0.0):
    lo, pl = _i32(out_size)
    hi, ph = _i32(out_size)
    d = np.zeros(out_size, dtype=np.float32)
    lib().orc_bilinear_table(I64(in_size), I64(out_size), I32(int(align)), F32(user_scale), pl, ph,
                             d.ctypes.data_as(ctypes.c_void_p))
    return lo, hi, d


def bilinear_bwd_table(in_size, out_size, align, user_scale=0.0):
    lo, pl = _i32(out_size)
    hi, ph = _i32(out_size)
    d = np.zeros(out_size, dtype=np.float32)
    lib().orc_bilinear_bwd_table(I64(in_size), I64(out_size), I32(int(align)), F32(user_scale), pl, ph,
                                 d.ctypes.data_as(ctypes.c_void_p))
    return lo, hi, d


def bicubic_aa_table(in_size, out_size, align, user_scale=0.0):
    fn = lib().orc_bicubic_aa_table
    fn.restype = ctypes.c_int32
    taps = max(1, fn(I64(in_size), I64(out_size), I32(int(align)), F32(user_scale), None, None, None, I32(0)))
    xmin, pm = _i32(out_size)
    xsize, ps = _i32(out_size)
    w = np.zeros((out_size, taps), dtype=np.float32)
    fn(I64(in_size), I64(out_size), I32(int(align)), F32(user_scale), pm, ps, w.ctypes.data_as(ctypes.c_void_p),
       I32(taps))
    return xmin, xsize, w


# ---- ops ---------------------------------------------------------------------------------------------------

def nearest2d_fwd(x, out_hw, scales=(0.0, 0.0), fmt=NCHW):
    x, px = _f(x)
    n, c, h, w = _dims(x.shape, fmt)
    y = np.empty(_shape(n, c, out_hw[0], out_hw[1], fmt), dtype=np.float32)
    lib().orc_nearest2d_fwd(px, y.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(h), I64(w), I64(out_hw[0]),
                            I64(out_hw[1]), F32(scales[0]), F32(scales[1]), I32(fmt))
    return y


def nearest2d_bwd(go, in_hw, scales=(0.0, 0.0), fmt=NCHW):
    go, pg = _f(go)
    n, c, ho, wo = _dims(go.shape, fmt)
    gi = np.empty(_shape(n, c, in_hw[0], in_hw[1], fmt), dtype=np.float32)
    lib().orc_nearest2d_bwd(pg, gi.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(in_hw[0]), I64(in_hw[1]),
                            I64(ho), I64(wo), F32(scales[0]), F32(scales[1]), I32(fmt))
    return gi


def nearest_exact_src_index(in_size, out_size, user_scale=0.0):
    idx, p = _i32(out_size)
    lib().orc_nearest_exact_src_index(I64(in_size), I64(out_size), F32(user_scale), p)
    return idx


def nearest_exact_bwd_ranges(in_size, out_size, user_scale=0.0):
    s, ps = _i32(in_size)
    e, pe = _i32(in_size)
    lib().orc_nearest_exact_bwd_ranges(I64(in_size), I64(out_size), F32(user_scale), ps, pe)
    return s, e


def nearest_exact2d_fwd(x, out_hw, scales=(0.0, 0.0), fmt=NCHW):
    x, px = _f(x)
    n, c, h, w = _dims(x.shape, fmt)
    y = np.empty(_shape(n, c, out_hw[0], out_hw[1], fmt), dtype=np.float32)
    lib().orc_nearest_exact2d_fwd(px, y.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(h), I64(w),
                                  I64(out_hw[0]), I64(out_hw[1]), F32(scales[0]), F32(scales[1]), I32(fmt))
    return y


def nearest_exact2d_bwd(go, in_hw, scales=(0.0, 0.0)):
    go, pg = _f(go)
    n, c, ho, wo = go.shape
    gi = np.empty((n, c, in_hw[0], in_hw[1]), dtype=np.float32)
    lib().orc_nearest_exact2d_bwd(pg, gi.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(in_hw[0]),
                                  I64(in_hw[1]), I64(ho), I64(wo), F32(scales[0]), F32(scales[1]))
    return gi


def _dims5(shape, fmt):
    if fmt == NHWC:  # NDHWC
        n, d, h, w, c = shape
    else:
        n, c, d, h, w = shape
    return int(n), int(c), int(d), int(h), int(w)


def _shape5(n, c, d, h, w, fmt):
    return (n, d, h, w, c) if fmt == NHWC else (n, c, d, h, w)


def nearest3d_fwd(x, out_dhw, scales=(0.0, 0.0, 0.0), exact=False, fmt=NCHW):
    """UpsampleNearest3d / UpsampleNearestExact3d forward; fmt NCHW means NCDHW, NHWC means NDHWC."""
    x, px = _f(x)
    n, c, d, h, w = _dims5(x.shape, fmt)
    y = np.empty(_shape5(n, c, *out_dhw, fmt), dtype=np.float32)
    lib().orc_nearest3d_fwd(px, y.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(d), I64(h), I64(w),
                            I64(out_dhw[0]), I64(out_dhw[1]), I64(out_dhw[2]), F32(scales[0]), F32(scales[1]),
                            F32(scales[2]), I32(int(exact)), I32(fmt))
    return y


def nearest3d_bwd(go, in_dhw, scales=(0.0, 0.0, 0.0), exact=False, fmt=NCHW):
    go, pg = _f(go)
    n, c, do, ho, wo = _dims5(go.shape, fmt)
    gi = np.empty(_shape5(n, c, *in_dhw, fmt), dtype=np.float32)
    lib().orc_nearest3d_bwd(pg, gi.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(in_dhw[0]), I64(in_dhw[1]),
                            I64(in_dhw[2]), I64(do), I64(ho), I64(wo), F32(scales[0]), F32(scales[1]), F32(scales[2]),
                            I32(int(exact)), I32(fmt))
    return gi


def trilinear3d_scale(in_size, out_size, align=False, scales=(0.0, 0.0, 0.0), axis=0):
    """Source-coordinate scale of one axis (0 D, 1 H, 2 W) as the reference's tiling computes it."""
    fn = lib().orc_trilinear3d_scale
    fn.restype = ctypes.c_float
    return float(fn(I64(in_size), I64(out_size), I32(int(align)), F64(scales[0]), F64(scales[1]), F64(scales[2]),
                    I32(axis)))


def trilinear3d_fwd_loop(in_dhw, out_dhw, align=False, scales=(0.0, 0.0, 0.0)):
    """Which loop of the reference's SIMT kernel the scales select."""
    fn = lib().orc_trilinear3d_fwd_loop
    fn.restype = ctypes.c_int
    k = fn(I64(in_dhw[0]), I64(in_dhw[1]), I64(in_dhw[2]), I64(out_dhw[0]), I64(out_dhw[1]), I64(out_dhw[2]),
           I32(int(align)), F64(scales[0]), F64(scales[1]), F64(scales[2]))
    return ("full", "d_only", "h_only", "w_only", "copy")[k]


def trilinear3d_fwd(x, out_dhw, align=False, scales=(0.0, 0.0, 0.0), fmt=NCHW):
    """UpsampleTrilinear3d forward; fmt NCHW means NCDHW, NHWC means NDHWC. `scales` are the API's (output per
    input) factors, used only when all three are positive."""
    x, px = _f(x)
    n, c, d, h, w = _dims5(x.shape, fmt)
    y = np.empty(_shape5(n, c, *out_dhw, fmt), dtype=np.float32)
    lib().orc_trilinear3d_fwd(px, y.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(d), I64(h), I64(w),
                              I64(out_dhw[0]), I64(out_dhw[1]), I64(out_dhw[2]), I32(int(align)), F64(scales[0]),
                              F64(scales[1]), F64(scales[2]), I32(fmt))
    return y


def trilinear3d_bwd(go, in_dhw, align=False, scales=(0.0, 0.0, 0.0), fmt=NCHW):
    """UpsampleTrilinear3dBackward: three separable fp32 stages (W, H, D), ascending grad_output order in each."""
    go, pg = _f(go)
    n, c, do, ho, wo = _dims5(go.shape, fmt)
    gi = np.empty(_shape5(n, c, *in_dhw, fmt), dtype=np.float32)
    lib().orc_trilinear3d_bwd(pg, gi.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(in_dhw[0]), I64(in_dhw[1]),
                              I64(in_dhw[2]), I64(do), I64(ho), I64(wo), I32(int(align)), F64(scales[0]),
                              F64(scales[1]), F64(scales[2]), I32(fmt))
    return gi


def bilinear2d_fwd(x, out_hw, align=False, scales=(0.0, 0.0), fmt=NCHW):
    x, px = _f(x)
    n, c, h, w = _dims(x.shape, fmt)
    y = np.empty(_shape(n, c, out_hw[0], out_hw[1], fmt), dtype=np.float32)
    lib().orc_bilinear2d_fwd(px, y.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(h), I64(w), I64(out_hw[0]),
                             I64(out_hw[1]), I32(int(align)), F32(scales[0]), F32(scales[1]), I32(fmt))
    return y


def bilinear2d_bwd_kernel_choice(in_hw, out_hw, align=False, scales=(0.0, 0.0), deterministic=False, mixed_dtype=False):
    """Which kernel the reference's tiling runs for an NCHW call: "scatter" (atomic), "gather" (determine) or
    "gather_scales" (determine_scales)."""
    fn = lib().orc_bilinear2d_bwd_kernel_choice
    fn.restype = ctypes.c_int
    k = fn(I64(in_hw[0]), I64(in_hw[1]), I64(out_hw[0]), I64(out_hw[1]), I32(int(align)), F32(scales[0]),
           F32(scales[1]), I32(int(deterministic)), I32(int(mixed_dtype)))
    return ("scatter", "gather", "gather_scales")[k]


def bilinear2d_bwd(go, in_hw, align=False, scales=(0.0, 0.0), fmt=NCHW, definition="scatter", deterministic=False,
                   mixed_dtype=False):
    """definition: "scatter" (the atomic kernel run serially), "gather" (determine), "gather_scales"
    (determine_scales, align_corners = false only) or "dispatch" (whichever of the three the reference's tiling
    selects for these arguments)."""
    go, pg = _f(go)
    n, c, ho, wo = _dims(go.shape, fmt)
    gi = np.empty(_shape(n, c, in_hw[0], in_hw[1], fmt), dtype=np.float32)
    if definition == "dispatch":
        definition = bilinear2d_bwd_kernel_choice(in_hw, (ho, wo), align, scales, deterministic, mixed_dtype)
    if definition == "gather_scales":
        assert not align
        lib().orc_bilinear2d_bwd_gather_scales(pg, gi.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(in_hw[0]),
                                               I64(in_hw[1]), I64(ho), I64(wo), F32(scales[0]), F32(scales[1]),
                                               I32(fmt))
        return gi
    fn = lib().orc_bilinear2d_bwd_scatter if definition == "scatter" else lib().orc_bilinear2d_bwd_gather
    fn(pg, gi.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(in_hw[0]), I64(in_hw[1]), I64(ho), I64(wo),
       I32(int(align)), F32(scales[0]), F32(scales[1]), I32(fmt))
    return gi


def bicubic_aa_fwd(x, out_hw, align=False, scales=(0.0, 0.0)):
    x, px = _f(x)
    n, c, h, w = x.shape
    y = np.empty((n, c, out_hw[0], out_hw[1]), dtype=np.float32)
    lib().orc_bicubic_aa_fwd(px, y.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(h), I64(w), I64(out_hw[0]),
                             I64(out_hw[1]), I32(int(align)), F32(scales[0]), F32(scales[1]))
    return y


def bicubic_aa_bwd(go, in_hw, align=False, scales=(0.0, 0.0), definition="scatter"):
    go, pg = _f(go)
    n, c, ho, wo = go.shape
    gi = np.empty((n, c, in_hw[0], in_hw[1]), dtype=np.float32)
    fn = lib().orc_bicubic_aa_bwd_scatter if definition == "scatter" else lib().orc_bicubic_aa_bwd_gather
    fn(pg, gi.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(in_hw[0]), I64(in_hw[1]), I64(ho), I64(wo),
       I32(int(align)), F32(scales[0]), F32(scales[1]))
    return gi


def bilinear_aa_table(in_size, out_size, align, user_scale=0.0):
    """(xmin, xsize, weights[out, taps]) of UpsampleBilinear2dAA for one axis."""
    fn = lib().orc_bilinear_aa_table
    fn.restype = ctypes.c_int32
    taps = max(1, fn(I64(in_size), I64(out_size), I32(int(align)), F32(user_scale), None, None, None, I32(0)))
    xmin, pm = _i32(out_size)
    xsize, ps = _i32(out_size)
    w = np.zeros((out_size, taps), dtype=np.float32)
    fn(I64(in_size), I64(out_size), I32(int(align)), F32(user_scale), pm, ps, w.ctypes.data_as(ctypes.c_void_p),
       I32(taps))
    return xmin, xsize, w


def bilinear_aa_fwd(x, out_hw, align=False, scales=(0.0, 0.0)):
    x, px = _f(x)
    n, c, h, w = x.shape
    y = np.empty((n, c, out_hw[0], out_hw[1]), dtype=np.float32)
    lib().orc_bilinear_aa_fwd(px, y.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(h), I64(w), I64(out_hw[0]),
                              I64(out_hw[1]), I32(int(align)), F32(scales[0]), F32(scales[1]))
    return y


def bilinear_aa_bwd(go, in_hw, align=False, scales=(0.0, 0.0), definition="scatter"):
    """definition: "scatter" (the atomic kernel run serially) or "gather" (the deterministic kernel)."""
    go, pg = _f(go)
    n, c, ho, wo = go.shape
    gi = np.empty((n, c, in_hw[0], in_hw[1]), dtype=np.float32)
    fn = lib().orc_bilinear_aa_bwd_scatter if definition == "scatter" else lib().orc_bilinear_aa_bwd_gather
    fn(pg, gi.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(in_hw[0]), I64(in_hw[1]), I64(ho), I64(wo),
       I32(int(align)), F32(scales[0]), F32(scales[1]))
    return gi


def bicubic2d_fwd_schedule(in_hw, out_hw, align=False, scales=(0.0, 0.0)):
    """The schedule the reference's tiling picks for UpsampleBicubic2d: "general", "copy", "one_input_pixel",
    "one_output_pixel" or "integer_positions"."""
    fn = lib().orc_bicubic2d_fwd_schedule
    fn.restype = ctypes.c_int
    k = fn(I64(in_hw[0]), I64(in_hw[1]), I64(out_hw[0]), I64(out_hw[1]), I32(int(align)), F32(scales[0]),
           F32(scales[1]))
    return ("general", "copy", "one_input_pixel", "one_output_pixel", "integer_positions")[k]


def bicubic2d_fwd(x, out_hw, align=False, scales=(0.0, 0.0), fmt=NCHW):
    x, px = _f(x)
    n, c, h, w = _dims(x.shape, fmt)
    y = np.empty(_shape(n, c, out_hw[0], out_hw[1], fmt), dtype=np.float32)
    lib().orc_bicubic2d_fwd(px, y.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(h), I64(w), I64(out_hw[0]),
                            I64(out_hw[1]), I32(int(align)), F32(scales[0]), F32(scales[1]), I32(fmt))
    return y


def bicubic2d_bwd_kernel_choice(in_hw, out_hw, align=False, scales=(0.0, 0.0), deterministic=False):
    """Which kernel the reference's tiling runs for UpsampleBicubic2dBackward: "copy", "scatter" (atomic) or
    "gather" (determine)."""
    fn = lib().orc_bicubic2d_bwd_kernel_choice
    fn.restype = ctypes.c_int
    k = fn(I64(in_hw[0]), I64(in_hw[1]), I64(out_hw[0]), I64(out_hw[1]), I32(int(align)), F32(scales[0]),
           F32(scales[1]), I32(int(deterministic)))
    return ("copy", "scatter", "gather")[k]


def bicubic2d_bwd(go, in_hw, align=False, scales=(0.0, 0.0), fmt=NCHW, definition="scatter", deterministic=False):
    """definition: "scatter" (the atomic kernel run serially), "gather" (the determine kernel) or "dispatch"
    (whichever the reference's tiling selects; equal extents copy under every definition)."""
    go, pg = _f(go)
    n, c, ho, wo = _dims(go.shape, fmt)
    gi = np.empty(_shape(n, c, in_hw[0], in_hw[1], fmt), dtype=np.float32)
    if definition == "dispatch":
        definition = bicubic2d_bwd_kernel_choice(in_hw, (ho, wo), align, scales, deterministic)
        definition = "scatter" if definition == "copy" else definition
    fn = lib().orc_bicubic2d_bwd_scatter if definition == "scatter" else lib().orc_bicubic2d_bwd_gather
    fn(pg, gi.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(in_hw[0]), I64(in_hw[1]), I64(ho), I64(wo),
       I32(int(align)), F32(scales[0]), F32(scales[1]), I32(fmt))
    return gi


def grid_sampler2d_coords(grid, in_hw, pad=ZEROS, align=False):
    grid, pg = _f(grid)
    ns = grid.size // 2
    ix = np.empty(ns, dtype=np.float32)
    iy = np.empty(ns, dtype=np.float32)
    lib().orc_grid_sampler2d_coords(pg, ix.ctypes.data_as(ctypes.c_void_p), iy.ctypes.data_as(ctypes.c_void_p),
                                    I64(ns), I32(in_hw[0]), I32(in_hw[1]), I32(pad), I32(int(align)))
    return ix, iy


def grid_sampler2d_fwd(x, grid, interp=BILINEAR, pad=ZEROS, align=False):
    x, px = _f(x)
    grid, pg = _f(grid)
    n, c, h, w = x.shape
    _, ho, wo, _ = grid.shape
    y = np.empty((n, c, ho, wo), dtype=np.float32)
    lib().orc_grid_sampler2d_fwd(px, pg, y.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I32(h), I32(w), I32(ho),
                                 I32(wo), I32(interp), I32(pad), I32(int(align)))
    return y


def grid_sampler2d_bwd(go, x, grid, interp=BILINEAR, pad=ZEROS, align=False):
    go, pgo = _f(go)
    x, px = _f(x)
    grid, pg = _f(grid)
    n, c, h, w = x.shape
    _, ho, wo, _ = grid.shape
    gi = np.empty_like(x)
    gg = np.empty_like(grid)
    lib().orc_grid_sampler2d_bwd(pgo, px, pg, gi.ctypes.data_as(ctypes.c_void_p), gg.ctypes.data_as(ctypes.c_void_p),
                                 I64(n), I64(c), I32(h), I32(w), I32(ho), I32(wo), I32(interp), I32(pad),
                                 I32(int(align)))
    return gi, gg


def grid_sampler2d_bwd_det_order(go, x_shape, grid, interp=BILINEAR, pad=ZEROS, align=False):
    """grad_input with the fp32 additions in the reference's deterministic replay order (256-sample step, tap,
    sample)."""
    go, pgo = _f(go)
    grid, pg = _f(grid)
    n, c, h, w = x_shape
    _, ho, wo, _ = grid.shape
    gi = np.empty(tuple(x_shape), dtype=np.float32)
    lib().orc_grid_sampler2d_bwd_det_order(pgo, pg, gi.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I32(h), I32(w),
                                           I32(ho), I32(wo), I32(interp), I32(pad), I32(int(align)))
    return gi


def grid_sampler3d_fwd(x, grid, pad=ZEROS, align=False):
    """GridSampler3D, bilinear: x (N, C, D, H, W), grid (N, Do, Ho, Wo, 3) -> (N, C, Do, Ho, Wo)."""
    x, px = _f(x)
    grid, pg = _f(grid)
    n, c, d, h, w = x.shape
    _, do, ho, wo, _ = grid.shape
    y = np.empty((n, c, do, ho, wo), dtype=np.float32)
    lib().orc_grid_sampler3d_fwd(px, pg, y.ctypes.data_as(ctypes.c_void_p), I64(n), I64(c), I64(d), I64(h), I64(w),
                                 I64(do), I64(ho), I64(wo), I32(pad), I32(int(align)))
    return y


def grid_sampler3d_bwd(go, x, grid, interp=BILINEAR, pad=ZEROS, align=False):
    """GridSampler3DGrad (bilinear or nearest): returns (grad_input, grad_grid); the scatter runs serially."""
    go, pgo = _f(go)
    x, px = _f(x)
    grid, pg = _f(grid)
    n, c, d, h, w = x.shape
    _, do, ho, wo, _ = grid.shape
    gi = np.empty_like(x)
    gg = np.empty_like(grid)
    lib().orc_grid_sampler3d_bwd(pgo, px, pg, gi.ctypes.data_as(ctypes.c_void_p), gg.ctypes.data_as(ctypes.c_void_p),
                                 I64(n), I64(c), I64(d), I64(h), I64(w), I64(do), I64(ho), I64(wo), I32(interp),
                                 I32(pad), I32(int(align)))
    return gi, gg
