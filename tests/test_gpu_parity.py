"""GPU parity: the CUDA library, called through its C ABI, against the CPU oracle on the same seeded inputs.

Bars (written into each assertion):
  * integer tables (source indices, window bounds), nearest forward, nearest-mode grid sampling: bit-exact;
  * fp32 interpolated values and gradients: rtol 1e-5 / atol 1e-6 (most kernels keep the oracle's operation
    order and are in fact bit-identical, which is asserted where it holds by construction);
  * fp16 / bf16: the fp32 result rounded once; at most 1 ulp of the output dtype from the rounded oracle value.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 1e-6
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def gen(seed):
    return torch.Generator().manual_seed(seed)


def ulp_diff(a, b):
    """Distance in units of the last place between two tensors of one 16-bit (or 32-bit) float dtype."""
    it = {torch.float16: torch.int16, torch.bfloat16: torch.int16, torch.float32: torch.int32}[a.dtype]
    ai, bi = a.contiguous().view(it).to(torch.int64), b.contiguous().view(it).to(torch.int64)
    sign = 1 << (15 if a.dtype != torch.float32 else 31)
    ai = torch.where(ai < 0, -(ai + sign) - 0, ai)  # map sign-magnitude to a monotone integer line
    bi = torch.where(bi < 0, -(bi + sign) - 0, bi)
    return (ai - bi).abs().max().item() if a.numel() else 0


def check(got, ref32, dtype, exact=False, rtol=RTOL, atol=ATOL):
    """got: device tensor of `dtype`; ref32: fp32 numpy oracle result (before the final rounding)."""
    got = got.detach().cpu()
    ref = torch.from_numpy(np.ascontiguousarray(ref32))
    assert got.shape == ref.shape
    if dtype == torch.float32:
        if exact:
            assert torch.equal(got, ref), f"max abs diff {(got - ref).abs().max().item()}"
        else:
            np.testing.assert_allclose(got.numpy(), ref.numpy(), rtol=rtol, atol=atol)
    else:
        want = ref.to(dtype)
        if exact:
            assert torch.equal(got, want)
        else:
            d = ulp_diff(got, want)
            assert d <= 1, f"{d} ulp of {dtype}"


def check_dispatched(got, ref_dispatch, ref_other, dtype, rtol=RTOL, atol=ATOL):
    """For an operator with two reference kernels that are two roundings of one formula (the scatter and the gather
    form of a backward pass). `ref_dispatch` is the kernel the reference's tiling runs for these arguments. The result
    must hold the fp32 bar against it; where the reference's own two kernels are further apart than that bar (their
    source positions carry different fp32 roundings once coordinates are large or the scale is not a power of two),
    the result may be as far from the dispatched kernel as the reference's other kernel is, and no further.
    Returns (largest |got - ref_dispatch|, largest spread between the two reference kernels)."""
    got32 = got.detach().cpu().float().numpy()
    a, b = np.ascontiguousarray(ref_dispatch), np.ascontiguousarray(ref_other)
    assert got32.shape == a.shape
    spread = np.abs(a - b)
    if dtype == torch.float32:
        err = np.abs(got32 - a)
        bound = atol + rtol * np.abs(a) + spread
        assert (err <= bound).all(), f"max excess {(err - bound).max()} (spread {spread.max()})"
        return float(err.max()) if err.size else 0.0, float(spread.max()) if spread.size else 0.0
    # 16-bit: at most 1 ulp from the rounded dispatched value, or (where the two reference kernels disagree by more
    # than that, which happens for results that cancel to nearly zero) within the spread of the two in fp32
    want = torch.from_numpy(a).to(dtype)
    g16 = got.detach().cpu()
    one_ulp = (torch.nextafter(want.float().abs(), torch.tensor(float("inf"))).to(dtype).float()
               - want.float().abs()).abs().numpy()  # spacing of the dtype at |want| (fp32 spacing if it rounds back)
    step = np.maximum(one_ulp, np.abs(want.float().numpy()) * (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10))
    err = np.abs(g16.float().numpy() - a)
    ok = err <= step + spread + atol
    assert ok.all(), f"max excess {(err - step - spread).max()} (spread {spread.max()})"
    return float(err.max()) if err.size else 0.0, float(spread.max()) if spread.size else 0.0


def quant(x, dtype):
    """Round an fp32 tensor to the storage dtype; returns (storage tensor, its exact fp32 value as numpy)."""
    xs = x.to(dtype)
    return xs, xs.float().numpy()


def nhwc(a):
    return np.ascontiguousarray(np.transpose(a, (0, 2, 3, 1)))


SHAPES = [
    # (N, C, Hin, Win, Hout, Wout)
    (1, 3, 64, 64, 128, 128),   # configs[0]
    (2, 8, 14, 14, 28, 28),     # exact 2x
    (2, 3, 7, 9, 15, 20),       # ragged up-scale
    (1, 4, 16, 24, 5, 7),       # down-scale
    (1, 2, 1, 1, 3, 5),         # 1x1 input
    (2, 2, 5, 6, 1, 1),         # 1x1 output
    (1, 1, 3, 1, 7, 1),         # one column
    (1, 5, 9, 8, 9, 16),        # one axis unchanged
    (1, 16, 6, 8, 12, 16),      # C multiple of 8 (NHWC vector path), W multiple of 8
]


# ---------------------------------------------------------------------------------------------------------------
# tables
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("sizes", [(64, 128), (56, 112), (7, 15), (16, 5), (1, 4), (5, 1), (1024, 224), (96, 96 * 3)])
def test_axis_tables_bit_exact(ops, oracle, sizes):
    i, o = sizes
    for scale in (0.0, 2.0, 1.7):
        src, _, _ = ops.debug_axis_table("nearest_fwd", i, o, user_scale=scale)
        assert np.array_equal(src, oracle.nearest_src_index(i, o, scale))
        s, e, _ = ops.debug_axis_table("nearest_bwd", i, o, user_scale=scale)
        rs, re = oracle.nearest_bwd_ranges(i, o, scale)
        assert np.array_equal(s, rs) and np.array_equal(e, re)
        for align in (False, True):
            lo, hi, d = ops.debug_axis_table("bilinear", i, o, align, scale)
            rlo, rhi, rd = oracle.bilinear_table(i, o, align, scale)
            assert np.array_equal(lo, rlo) and np.array_equal(hi, rhi)
            assert np.array_equal(d.view(np.int32), rd.view(np.int32))  # fp32 weights bit for bit
            xmin, xsize, w = ops.debug_axis_table("bicubic_aa", i, o, align, scale)
            rmin, rsize, rw = oracle.bicubic_aa_table(i, o, align, scale)
            assert np.array_equal(xmin, rmin) and np.array_equal(xsize, rsize)
            assert w.shape[1] >= rw.shape[1]
            assert np.array_equal(w[:, :rw.shape[1]].view(np.int32), rw.view(np.int32))
            assert not w[:, rw.shape[1]:].any()


# ---------------------------------------------------------------------------------------------------------------
# nearest
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("fmt", ["NCHW", "NHWC"])
@pytest.mark.parametrize("shape", SHAPES)
def test_nearest_forward_backward(ops, oracle, dev, dtype, fmt, shape):
    n, c, hi, wi, ho, wo = shape
    x, x32 = quant(torch.randn((n, c, hi, wi), generator=gen(1)), dtype)
    g, g32 = quant(torch.randn((n, c, ho, wo), generator=gen(2)), dtype)
    f = oracle.NCHW if fmt == "NCHW" else oracle.NHWC
    if fmt == "NHWC":
        x, x32 = x.permute(0, 2, 3, 1).contiguous(), nhwc(x32)
        g, g32 = g.permute(0, 2, 3, 1).contiguous(), nhwc(g32)
    y = ops.upsample_nearest2d(x.to(dev), (ho, wo), fmt)
    check(y, oracle.nearest2d_fwd(x32, (ho, wo), fmt=f), dtype, exact=True)
    gi = ops.upsample_nearest2d_backward(g.to(dev), (ho, wo), tuple(x.shape), fmt)
    check(gi, oracle.nearest2d_bwd(g32, (hi, wi), fmt=f), dtype, exact=True)  # same fp32 summation order


def test_nearest_v2_user_scales(ops, oracle, dev):
    x = torch.randn((1, 2, 5, 6), generator=gen(3))
    y = ops.upsample_nearest2d(x.to(dev), (12, 16), scales=(2.5, 2.7))
    check(y, oracle.nearest2d_fwd(x.numpy(), (12, 16), (2.5, 2.7)), torch.float32, exact=True)
    g = torch.randn((1, 2, 12, 16), generator=gen(4))
    gi = ops.upsample_nearest2d_backward(g.to(dev), (12, 16), (1, 2, 5, 6), scales=(2.5, 2.7))
    check(gi, oracle.nearest2d_bwd(g.numpy(), (5, 6), (2.5, 2.7)), torch.float32, exact=True)


# ---------------------------------------------------------------------------------------------------------------
# bilinear
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("fmt", ["NCHW", "NHWC"])
@pytest.mark.parametrize("align", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_bilinear_forward(ops, oracle, dev, dtype, fmt, align, shape):
    n, c, hi, wi, ho, wo = shape
    x, x32 = quant(torch.randn((n, c, hi, wi), generator=gen(5)), dtype)
    f = oracle.NCHW if fmt == "NCHW" else oracle.NHWC
    if fmt == "NHWC":
        x, x32 = x.permute(0, 2, 3, 1).contiguous(), nhwc(x32)
    y = ops.upsample_bilinear2d(x.to(dev), (ho, wo), align, fmt)
    check(y, oracle.bilinear2d_fwd(x32, (ho, wo), align, fmt=f), dtype, exact=True)  # same operation order


NHWC_X2_SHAPES = [
    # (N, C, Hin, Win): NHWC, output (2 Hin, 2 Win); C a multiple of 8 so that 16-bit tensors take 16-byte vectors
    (1, 8, 1, 1),
    (2, 8, 2, 3),
    (1, 16, 3, 5),
    (1, 8, 8, 8),
    (2, 24, 33, 7),    # an odd number of steps, several row chunks
    (1, 8, 130, 2),    # a long walk cut into chunks of steps
    (64, 32, 6, 40),   # enough walkers for one chunk per column
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", NHWC_X2_SHAPES)
def test_bilinear_forward_nhwc_2x_walk(ops, oracle, dev, dtype, shape):
    """The straight-line 2x row walk of the NHWC kernel (with and without user scales): the oracle's bits."""
    n, c, hi, wi = shape
    x, x32 = quant(torch.randn((n, c, hi, wi), generator=gen(160)), dtype)
    xl, x32l = x.permute(0, 2, 3, 1).contiguous(), nhwc(x32)
    for scales in ((0.0, 0.0), (2.0, 2.0)):
        y = ops.upsample_bilinear2d(xl.to(dev), (2 * hi, 2 * wi), False, "NHWC", scales=scales)
        check(y, oracle.bilinear2d_fwd(x32l, (2 * hi, 2 * wi), False, scales, fmt=oracle.NHWC), dtype, exact=True)
    xs = x32l.copy()
    xs[0, 0, 0, 0] = np.inf
    xs[-1, -1, -1, -1] = np.nan
    ys = ops.upsample_bilinear2d(torch.from_numpy(xs).to(dtype).to(dev), (2 * hi, 2 * wi), False, "NHWC").float().cpu().numpy()
    ref = oracle.bilinear2d_fwd(xs, (2 * hi, 2 * wi), False, fmt=oracle.NHWC)
    assert np.array_equal(np.isnan(ys), np.isnan(ref)) and np.array_equal(np.isinf(ys), np.isinf(ref))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("fmt", ["NCHW", "NHWC"])
@pytest.mark.parametrize("align", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_bilinear_backward_gather(ops, oracle, dev, dtype, fmt, align, shape):
    n, c, hi, wi, ho, wo = shape
    g, g32 = quant(torch.randn((n, c, ho, wo), generator=gen(6)), dtype)
    f = oracle.NCHW if fmt == "NCHW" else oracle.NHWC
    in_shape = (n, c, hi, wi)
    if fmt == "NHWC":
        g, g32 = g.permute(0, 2, 3, 1).contiguous(), nhwc(g32)
        in_shape = (n, hi, wi, c)
    scatter = oracle.bilinear2d_bwd(g32, (hi, wi), align, fmt=f, definition="scatter")
    # the kernel the reference's tiling runs: the gather ("determine") kernel for every up-scale, with or without
    # the deterministic option; the atomic scatter for down-scales when the option is off
    dispatched = oracle.bilinear2d_bwd(g32, (hi, wi), align, fmt=f, definition="dispatch")
    exact_ratio = not align and ho % hi == 0 and wo % wi == 0
    for v2 in (False, True):
        gi = ops.upsample_bilinear2d_backward(g.to(dev), (ho, wo), in_shape, align, fmt, v2=v2)
        # NHWC: the gather adds the scatter kernel's products in the serial scatter order: identical to that
        # oracle. NCHW: separable row walk with fused multiply-adds, fixed order: within tolerance (<= 1 ulp 16-bit).
        check(gi, scatter, dtype, exact=(fmt == "NHWC"))
        if exact_ratio:
            # integer ratios (cfg2's 2x among them): source positions are exact in fp32 in both reference kernels, so
            # the bar holds against the dispatched kernel with no allowance
            check(gi, dispatched, dtype)
        else:
            check_dispatched(gi, dispatched, scatter, dtype)
        gi_again = ops.upsample_bilinear2d_backward(g.to(dev), (ho, wo), in_shape, align, fmt, v2=v2)
        assert torch.equal(gi.cpu().view(torch.uint8), gi_again.cpu().view(torch.uint8))  # reproducible


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("fmt", ["NCHW", "NHWC"])
def test_bilinear_backward_atomic_mode(ops, oracle, dev, dtype, fmt):
    n, c, hi, wi, ho, wo = 2, 8, 14, 12, 28, 24
    g, g32 = quant(torch.randn((n, c, ho, wo), generator=gen(7)), dtype)
    f = oracle.NCHW if fmt == "NCHW" else oracle.NHWC
    in_shape = (n, c, hi, wi)
    if fmt == "NHWC":
        g, g32 = g.permute(0, 2, 3, 1).contiguous(), nhwc(g32)
        in_shape = (n, hi, wi, c)
    ops.set_backward_algo("atomic")
    try:
        gi = ops.upsample_bilinear2d_backward(g.to(dev), (ho, wo), in_shape, False, fmt)
    finally:
        ops.set_backward_algo("gather")
    check(gi, oracle.bilinear2d_bwd(g32, (hi, wi), False, fmt=f), dtype)


def test_bilinear_user_scales_and_mixed_dtype(ops, oracle, dev):
    x = torch.randn((1, 2, 8, 8), generator=gen(8))
    y = ops.upsample_bilinear2d(x.to(dev), (16, 16), False, scales=(2.0, 2.0))
    check(y, oracle.bilinear2d_fwd(x.numpy(), (16, 16), False, (2.0, 2.0)), torch.float32, exact=True)
    # user scales that disagree with the size ratio (the reference's "determine_scales" situation)
    g = torch.randn((1, 2, 20, 22), generator=gen(9))
    gi = ops.upsample_bilinear2d_backward(g.to(dev), (20, 22), (1, 2, 8, 8), False, scales=(2.0, 2.0))
    check(gi, oracle.bilinear2d_bwd(g.numpy(), (8, 8), False, (2.0, 2.0)), torch.float32, exact=True)
    for sc in ((2.0, 2.0), (2.4, 2.9), (3.0, 1.5)):
        assert oracle.bilinear2d_bwd_kernel_choice((8, 8), (20, 22), False, sc) == "gather_scales"
        gi = ops.upsample_bilinear2d_backward(g.to(dev), (20, 22), (1, 2, 8, 8), False, scales=sc)
        # the kernel the reference runs here recomputes every source position from the user scale and treats the
        # border rows and columns separately (resize_bilinear_v2_grad_simt_determine_scales.h:61-250)
        check(gi, oracle.bilinear2d_bwd(g.numpy(), (8, 8), False, sc, definition="gather_scales"), torch.float32)
    # fp32 grads -> bf16 gradient
    gi16 = ops.upsample_bilinear2d_backward(g.to(dev), (20, 22), (1, 2, 8, 8), False, out_dtype=torch.bfloat16)
    check(gi16, oracle.bilinear2d_bwd(g.numpy(), (8, 8), False), torch.bfloat16)


# ---------------------------------------------------------------------------------------------------------------
# bicubic, anti-aliased
# ---------------------------------------------------------------------------------------------------------------
AA_SHAPES = [(1, 2, 32, 40, 7, 9), (2, 3, 64, 64, 14, 14), (1, 2, 6, 7, 13, 15), (1, 1, 9, 9, 9, 4),
             (1, 3, 128, 96, 28, 21), (1, 1, 5, 5, 1, 1), (1, 2, 1, 1, 4, 4), (1, 1, 40, 3, 8, 3)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("align", [False, True])
@pytest.mark.parametrize("shape", AA_SHAPES)
def test_bicubic_aa_forward(ops, oracle, dev, dtype, align, shape):
    n, c, hi, wi, ho, wo = shape
    x, x32 = quant(torch.rand((n, c, hi, wi), generator=gen(10)), dtype)
    y = ops.upsample_bicubic2d_aa(x.to(dev), (ho, wo), align)
    check(y, oracle.bicubic_aa_fwd(x32, (ho, wo), align), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("align", [False, True])
@pytest.mark.parametrize("shape", AA_SHAPES)
@pytest.mark.parametrize("algo", ["gather", "atomic"])
def test_bicubic_aa_backward(ops, oracle, dev, dtype, align, shape, algo):
    n, c, hi, wi, ho, wo = shape
    g, g32 = quant(torch.randn((n, c, ho, wo), generator=gen(11)), dtype)
    ops.set_backward_algo(algo)
    try:
        gi = ops.upsample_bicubic2d_aa_grad(g.to(dev), (ho, wo), (n, c, hi, wi), align)
    finally:
        ops.set_backward_algo("gather")
    ref = oracle.bicubic_aa_bwd(g32, (hi, wi), align, definition="scatter")
    check(gi, ref, dtype)
    # The reference's deterministic kernel is a second formulation of the same gradient. The two agree except when
    # the scale is 0 (align_corners with a single output pixel), where they place the filter centre differently;
    # the library follows the kernel the mode selects.
    ops.set_deterministic(True)
    try:
        gd = ops.upsample_bicubic2d_aa_grad(g.to(dev), (ho, wo), (n, c, hi, wi), align)
        gd2 = ops.upsample_bicubic2d_aa_grad(g.to(dev), (ho, wo), (n, c, hi, wi), align)
    finally:
        ops.set_deterministic(False)
    assert torch.equal(gd, gd2)
    rd = oracle.bicubic_aa_bwd(g32, (hi, wi), align, definition="gather")
    if dtype == torch.float32:
        np.testing.assert_allclose(gd.cpu().numpy(), rd, rtol=1e-4, atol=1e-5)
    degenerate = align and (ho == 1 or wo == 1)
    if not degenerate and dtype == torch.float32:
        np.testing.assert_allclose(gi.cpu().numpy(), rd, rtol=1e-4, atol=1e-5)


def test_bicubic_aa_user_scales(ops, oracle, dev):
    x = torch.rand((1, 2, 20, 24), generator=gen(12))
    y = ops.upsample_bicubic2d_aa(x.to(dev), (10, 8), False, scales=(0.5, 1.0 / 3.0))
    check(y, oracle.bicubic_aa_fwd(x.numpy(), (10, 8), False, (0.5, 1.0 / 3.0)), torch.float32)
    g = torch.randn((1, 2, 10, 8), generator=gen(13))
    gi = ops.upsample_bicubic2d_aa_grad(g.to(dev), (10, 8), (1, 2, 20, 24), False, scales=(0.5, 1.0 / 3.0))
    check(gi, oracle.bicubic_aa_bwd(g.numpy(), (20, 24), False, (0.5, 1.0 / 3.0)), torch.float32)


# ---------------------------------------------------------------------------------------------------------------
# grid sampler
# ---------------------------------------------------------------------------------------------------------------
def make_grid(n, ho, wo, seed, span=1.1):
    return torch.rand((n, ho, wo, 2), generator=gen(seed)) * (2 * span) - span


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("interp", [0, 1, 2])
@pytest.mark.parametrize("pad", [0, 1, 2])
@pytest.mark.parametrize("align", [False, True])
def test_grid_sampler_forward(ops, oracle, dev, dtype, interp, pad, align):
    n, c, hi, wi, ho, wo = 2, 5, 9, 11, 6, 7
    x, x32 = quant(torch.randn((n, c, hi, wi), generator=gen(20)), dtype)
    grid, grid32 = quant(make_grid(n, ho, wo, 21, 1.3), dtype)
    y = ops.grid_sampler2d(x.to(dev), grid.to(dev), interp, pad, align)
    # same operation order as the oracle: the fp32 result is identical
    check(y, oracle.grid_sampler2d_fwd(x32, grid32, interp, pad, align), dtype, exact=True)


def test_grid_sampler_forward_special_values(ops, oracle, dev):
    x = torch.randn((1, 3, 4, 5), generator=gen(22))
    grid = make_grid(1, 3, 4, 23)
    grid[0, 0, 0, 0] = float("nan")
    grid[0, 0, 1, 1] = float("inf")
    grid[0, 1, 0, 0] = -float("inf")
    grid[0, 1, 1] = torch.tensor([1e10, -1e10])
    grid[0, 2, 0] = torch.tensor([-1.0, 1.0])
    for interp in (0, 1):
        for pad in (0, 1, 2):
            y = ops.grid_sampler2d(x.to(dev), grid.to(dev), interp, pad, False).cpu().numpy()
            ref = oracle.grid_sampler2d_fwd(x.numpy(), grid.numpy(), interp, pad, False)
            assert np.array_equal(np.isnan(y), np.isnan(ref)), (interp, pad)
            assert np.array_equal(np.nan_to_num(y), np.nan_to_num(ref)), (interp, pad)


def affine_grid(n, ho, wo, seed, max_deg=30.0, scale=(0.8, 1.2), shift=0.1):
    g = gen(seed)
    phi = (torch.rand(n, generator=g) * 2 - 1) * max_deg * np.pi / 180
    s = torch.rand(n, generator=g) * (scale[1] - scale[0]) + scale[0]
    t = (torch.rand((n, 2), generator=g) * 2 - 1) * shift
    theta = torch.stack([torch.stack([s * torch.cos(phi), -s * torch.sin(phi), t[:, 0]], 1),
                         torch.stack([s * torch.sin(phi), s * torch.cos(phi), t[:, 1]], 1)], 1)
    return torch.nn.functional.affine_grid(theta, (n, 1, ho, wo), align_corners=False).contiguous()


@pytest.mark.parametrize("pad", [0, 1, 2])
@pytest.mark.parametrize("align", [False, True])
@pytest.mark.parametrize("case", ["affine", "random", "mixed", "far"])
def test_grid_sampler_forward_large_planes(ops, oracle, dev, pad, align, case):
    """fp32 planes too large for the plane-major staged kernel take the tile-major kernel that stages, per 32 x 32
    output tile, the window of the input its taps fall into. Smooth grids (affine) stay in shared memory; a random
    grid makes every tile fall back to global-memory taps; "mixed" has both kinds of tile plus NaN / Inf samples; "far"
    puts a whole tile outside the image. C = 6 leaves a partial last channel group; the output is not a multiple of
    the tile. Same operation order as the oracle: identical bits."""
    n, c, hi, wi, ho, wo = 2, 6, 100, 92, 110, 85
    x = torch.randn((n, c, hi, wi), generator=gen(50))
    if case == "affine":
        grid = affine_grid(n, ho, wo, 51)
    elif case == "random":
        grid = make_grid(n, ho, wo, 52, 1.2)
    elif case == "mixed":
        grid = affine_grid(n, ho, wo, 53, 45.0, (0.5, 1.5), 0.3)
        grid[1, 40:70, :20] = make_grid(1, 30, 20, 54, 1.3)[0]
        grid[0, 3, 4, 0] = float("nan")
        grid[0, 50, 40, 1] = float("inf")
        grid[1, 109, 84] = torch.tensor([-float("inf"), 0.2])
    else:
        grid = affine_grid(n, ho, wo, 55, 10.0, (0.9, 1.1), 0.05)
        grid[0, :32, :32] += 5.0   # a tile whose taps all miss the image
        grid[1, 32:64, :32, 0] = 1e30
    y = ops.grid_sampler2d(x.to(dev), grid.to(dev), 0, pad, align).cpu().numpy()
    ref = oracle.grid_sampler2d_fwd(x.numpy(), grid.numpy(), 0, pad, align)
    assert np.array_equal(np.isnan(y), np.isnan(ref))
    assert np.array_equal(np.nan_to_num(y).view(np.int32), np.nan_to_num(ref).view(np.int32))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("interp", [0, 1, 2])
@pytest.mark.parametrize("pad", [0, 1, 2])
@pytest.mark.parametrize("align", [False, True])
@pytest.mark.parametrize("det", [False, True])
def test_grid_sampler_backward(ops, oracle, dev, dtype, interp, pad, align, det):
    n, c, hi, wi, ho, wo = 2, 5, 9, 11, 12, 23
    x, x32 = quant(torch.randn((n, c, hi, wi), generator=gen(24)), dtype)
    grid, grid32 = quant(make_grid(n, ho, wo, 25, 1.2), dtype)
    g, g32 = quant(torch.randn((n, c, ho, wo), generator=gen(26)), dtype)
    ops.set_deterministic(det)
    try:
        gi, gg = ops.grid_sampler2d_backward(g.to(dev), x.to(dev), grid.to(dev), interp, pad, align)
        if det:
            gi2, gg2 = ops.grid_sampler2d_backward(g.to(dev), x.to(dev), grid.to(dev), interp, pad, align)
            assert torch.equal(gi.view(torch.int16 if dtype != torch.float32 else torch.int32),
                               gi2.view(torch.int16 if dtype != torch.float32 else torch.int32))
            assert torch.equal(gg, gg2) or (torch.isnan(gg) == torch.isnan(gg2)).all()
    finally:
        ops.set_deterministic(False)
    ri, rg = oracle.grid_sampler2d_bwd(g32, x32, grid32, interp, pad, align)
    check(gi, ri, dtype)
    check(gg, rg, dtype, exact=True)  # per-sample channel sum in channel order, as the oracle
    if det:  # the reproducible mode replays the reference's deterministic order: the same bits as a serial replay
        check(gi, oracle.grid_sampler2d_bwd_det_order(g32, x32.shape, grid32, interp, pad, align), dtype, exact=True)



def check_sum(got, ref32, dtype):
    """For values that are long sums evaluated in a different order than the oracle's (atomics, partial sums):
    relative tolerance of the dtype plus an absolute term scaled by the largest magnitude, because a sum that
    cancels to nearly zero carries the rounding of its large terms."""
    got = got.detach().cpu().float().numpy()
    ref = np.ascontiguousarray(ref32)
    assert got.shape == ref.shape
    assert np.array_equal(np.isnan(got), np.isnan(ref))
    scale = float(np.nanmax(np.abs(ref))) if ref.size else 0.0
    rel = {torch.float32: 1e-5, torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7}[dtype]
    abs_ = (1e-6 if dtype == torch.float32 else rel * 1e-2) * max(scale, 1.0)
    np.testing.assert_allclose(np.nan_to_num(got), np.nan_to_num(ref), rtol=rel, atol=abs_)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pad", [0, 1, 2])
@pytest.mark.parametrize("align", [False, True])
@pytest.mark.parametrize("c", [80, 161])
def test_grid_sampler_staged_kernels(ops, oracle, dev, dtype, pad, align, c):
    """Enough (image, channel group) blocks for the shared-memory staged kernels of the bilinear forward and the
    atomic-mode backward; c = 161 leaves a partial last group."""
    n, hi, wi, ho, wo = 8, 9, 11, 14, 13
    x, x32 = quant(torch.randn((n, c, hi, wi), generator=gen(40)), dtype)
    grid, grid32 = quant(make_grid(n, ho, wo, 41, 1.2), dtype)
    g, g32 = quant(torch.randn((n, c, ho, wo), generator=gen(42)), dtype)
    y = ops.grid_sampler2d(x.to(dev), grid.to(dev), 0, pad, align)
    check(y, oracle.grid_sampler2d_fwd(x32, grid32, 0, pad, align), dtype, exact=(dtype == torch.float32))
    ri, rg = oracle.grid_sampler2d_bwd(g32, x32, grid32, 0, pad, align)
    gi, gg = ops.grid_sampler2d_backward(g.to(dev), x.to(dev), grid.to(dev), 0, pad, align)
    check_sum(gi, ri, dtype)
    check_sum(gg, rg, dtype)
    # reproducible mode: chunked segment lists + staged gather, grad_grid from per-group partial sums
    ops.set_deterministic(True)
    try:
        runs = [ops.grid_sampler2d_backward(g.to(dev), x.to(dev), grid.to(dev), 0, pad, align) for _ in range(2)]
        only_grid = ops.grid_sampler2d_backward(g.to(dev), x.to(dev), grid.to(dev), 0, pad, align, mask=(False, True))
    finally:
        ops.set_deterministic(False)
    bits = torch.int32 if dtype == torch.float32 else torch.int16
    assert torch.equal(runs[0][0].view(bits), runs[1][0].view(bits))
    assert torch.equal(runs[0][1].view(bits), runs[1][1].view(bits))
    assert torch.equal(runs[0][1].view(bits), only_grid[1].view(bits))
    check_sum(runs[0][0], ri, dtype)
    check_sum(runs[0][1], rg, dtype)
    sentinel = torch.full_like(x, 7.0).to(dev)
    gi3, gg3 = ops.grid_sampler2d_backward(g.to(dev), x.to(dev), grid.to(dev), 0, pad, align, mask=(False, True),
                                           input_grad=sentinel)
    assert torch.equal(gi3.cpu(), torch.full_like(x, 7.0))
    check_sum(gg3, rg, dtype)
    sentinel_g = torch.full_like(grid, 7.0).to(dev)
    gi4, gg4 = ops.grid_sampler2d_backward(g.to(dev), x.to(dev), grid.to(dev), 0, pad, align, mask=(True, False),
                                           grid_grad=sentinel_g)
    assert torch.equal(gg4.cpu(), torch.full_like(grid, 7.0))
    check_sum(gi4, ri, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("interp", [0, 1, 2])
@pytest.mark.parametrize("shape", [(2, 5, 9, 11, 12, 23), (3, 4, 16, 16, 40, 37), (8, 80, 9, 11, 30, 29)])
def test_grid_sampler_backward_deterministic_order(ops, oracle, dev, dtype, interp, shape):
    """The reproducible mode adds the contributions of a destination in the order of the reference's deterministic
    kernel (256-sample steps; inside a step tap NW, NE, SW, SE; inside a tap ascending sample), so grad_input equals
    a serial replay in that order bit for bit. Shapes: one and several steps per image, heavy collisions (a coarse
    4-pixel grid of destinations), and enough blocks for the staged gather."""
    n, c, hi, wi, ho, wo = shape
    grid, grid32 = quant(make_grid(n, ho, wo, 71, 1.15), dtype)
    if shape[1] == 4:  # many samples per destination
        grid = (grid * 2).round() / 2
        grid, grid32 = quant(grid.float(), dtype)
    g, g32 = quant(torch.randn((n, c, ho, wo), generator=gen(72)), dtype)
    x = torch.zeros((n, c, hi, wi), dtype=dtype)
    ops.set_deterministic(True)
    try:
        gi, _ = ops.grid_sampler2d_backward(g.to(dev), x.to(dev), grid.to(dev), interp, 0, False, mask=(True, False))
    finally:
        ops.set_deterministic(False)
    ref = oracle.grid_sampler2d_bwd_det_order(g32, (n, c, hi, wi), grid32, interp, 0, False)
    check(gi, ref, dtype, exact=True)


def test_grid_sampler_backward_masks_and_collisions(ops, oracle, dev):
    # every sample hits the same source pixel: worst case for atomics and for the deterministic segment lists
    n, c, hi, wi, ho, wo = 1, 3, 4, 4, 40, 37
    x = torch.randn((n, c, hi, wi), generator=gen(27))
    grid = torch.zeros((n, ho, wo, 2)) + 0.01
    g = torch.randn((n, c, ho, wo), generator=gen(28))
    ri, rg = oracle.grid_sampler2d_bwd(g.numpy(), x.numpy(), grid.numpy())
    for det in (False, True):
        ops.set_deterministic(det)
        try:
            gi, gg = ops.grid_sampler2d_backward(g.to(dev), x.to(dev), grid.to(dev))
            np.testing.assert_allclose(gi.cpu().numpy(), ri, rtol=1e-4, atol=1e-4)
            assert np.array_equal(gg.cpu().numpy(), rg)
            # masks: an unrequested output is left untouched
            sentinel = torch.full_like(x, 7.0).to(dev)
            gi3, gg3 = ops.grid_sampler2d_backward(g.to(dev), x.to(dev), grid.to(dev), mask=(False, True),
                                                   input_grad=sentinel)
            assert torch.equal(gi3.cpu(), torch.full_like(x, 7.0)) and np.array_equal(gg3.cpu().numpy(), rg)
            sentinel_g = torch.full_like(grid, 7.0).to(dev)
            gi4, gg4 = ops.grid_sampler2d_backward(g.to(dev), x.to(dev), grid.to(dev), mask=(True, False),
                                                   grid_grad=sentinel_g)
            assert torch.equal(gg4.cpu(), torch.full_like(grid, 7.0))
            np.testing.assert_allclose(gi4.cpu().numpy(), ri, rtol=1e-4, atol=1e-4)
        finally:
            ops.set_deterministic(False)


# ---------------------------------------------------------------------------------------------------------------
# views, empties, golden fixtures
# ---------------------------------------------------------------------------------------------------------------
def test_strided_views(ops, oracle, dev):
    base = torch.randn((2, 3, 10, 24), generator=gen(30)).to(dev)
    x = base[:, :, 1:8, ::2]  # non-contiguous input view
    assert not x.is_contiguous()
    out_base = torch.zeros((2, 3, 14, 48), device=dev)
    out = out_base[:, :, :, ::2]  # non-contiguous output view
    ops.upsample_bilinear2d(x, (14, 24), False, out=out)
    ref = oracle.bilinear2d_fwd(x.cpu().numpy(), (14, 24), False)
    assert np.array_equal(out.cpu().numpy(), ref)
    assert not out_base[:, :, :, 1::2].any()  # the gaps of the view are untouched
    # channels-last storage passed as an NCHW view (strides (HWC, 1, WC, C))
    xc = torch.randn((2, 4, 6, 5), generator=gen(31)).to(dev).contiguous(memory_format=torch.channels_last)
    y = ops.upsample_nearest2d(xc, (12, 10))
    assert np.array_equal(y.cpu().numpy(), oracle.nearest2d_fwd(xc.cpu().numpy(), (12, 10)))
    grid = make_grid(2, 3, 4, 32).to(dev)
    gs = ops.grid_sampler2d(xc, grid)
    assert np.array_equal(gs.cpu().numpy(), oracle.grid_sampler2d_fwd(xc.cpu().numpy(), grid.cpu().numpy()))


def test_empty_tensors_are_noops(ops, dev):
    x = torch.zeros((0, 3, 4, 5), device=dev)
    assert ops.upsample_nearest2d(x, (8, 10)).shape == (0, 3, 8, 10)
    assert ops.upsample_bilinear2d(x, (8, 10)).shape == (0, 3, 8, 10)
    assert ops.upsample_bicubic2d_aa(x, (2, 2)).shape == (0, 3, 2, 2)
    assert ops.grid_sampler2d(x, torch.zeros((0, 2, 2, 2), device=dev)).shape == (0, 3, 2, 2)
    before = ops.launch_count()
    ops.upsample_nearest2d(x, (8, 10))
    assert ops.launch_count() == before


def test_golden_fixtures_on_gpu(ops, dev):
    """The committed reference goldens (see tests/golden/make_golden.py), at the reference tests' own tolerance."""
    import ast
    import os
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "resample_golden.npz"))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
    for m in gold["meta.interp"]:
        name, mode, shape, out, align, scales = ast.literal_eval(str(m))
        sc = scales if scales is not None else (0.0, 0.0)
        x, g = t(gold[name + ".x"]), t(gold[name + ".g"])
        if mode == "nearest":
            y = ops.upsample_nearest2d(x, out, scales=None if scales is None else sc)
            gx = ops.upsample_nearest2d_backward(g, out, shape, scales=sc)
        elif name.startswith("bilinear"):
            y = ops.upsample_bilinear2d(x, out, align, scales=sc)
            gx = ops.upsample_bilinear2d_backward(g, out, shape, align, scales=sc)
        else:
            y = ops.upsample_bicubic2d_aa(x, out, align, scales=sc)
            gx = ops.upsample_bicubic2d_aa_grad(g, out, shape, align, scales=sc)
        np.testing.assert_allclose(y.cpu().numpy(), gold[name + ".y"], rtol=1e-4, atol=1e-5, err_msg=name)
        np.testing.assert_allclose(gx.cpu().numpy(), gold[name + ".gx"], rtol=1e-4, atol=2e-5, err_msg=name)
    for mi, mode in enumerate(["bilinear", "nearest", "bicubic"]):
        for pi, pad in enumerate(["zeros", "border", "reflection"]):
            for align in (False, True):
                name = f"grid.{mode}.{pad}.{'ac' if align else 'hp'}"
                x, grid = t(gold[name + ".x"]), t(gold[name + ".grid"])
                y = ops.grid_sampler2d(x, grid, mi, pi, align)
                np.testing.assert_allclose(y.cpu().numpy(), gold[name + ".y"], rtol=1e-4, atol=1e-5, err_msg=name)
                if mode != "bicubic":
                    gi, gg = ops.grid_sampler2d_backward(t(gold[name + ".g"]), x, grid, mi, pi, align)
                    np.testing.assert_allclose(gi.cpu().numpy(), gold[name + ".gx"], rtol=1e-4, atol=1e-5)
                    np.testing.assert_allclose(gg.cpu().numpy(), gold[name + ".ggrid"], rtol=1e-3, atol=1e-4)
    y = ops.upsample_bilinear2d(t(gold["example.bilinear.x"]), (8, 4), True, scales=(2.0, 2.0))
    np.testing.assert_allclose(y.cpu().numpy(), gold["example.bilinear.y"], rtol=1e-5, atol=1e-6)


def test_second_phase_consumes_executor(ops, dev):
    import ctypes
    L = ops.lib()
    x = torch.randn((1, 1, 4, 4), device=dev)
    y = torch.empty((1, 1, 8, 8), device=dev)
    tx, ty, sz = ops.acl_tensor(x), ops.acl_tensor(y), ops.int_array([8, 8])
    ws, ex = ctypes.c_uint64(0), ctypes.c_void_p(None)
    assert L.aclnnUpsampleNearest2dGetWorkspaceSize(tx.ptr, sz.ptr, ty.ptr, ctypes.byref(ws), ctypes.byref(ex)) == 0
    buf = torch.empty(ws.value, dtype=torch.uint8, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.aclnnUpsampleNearest2d(ctypes.c_void_p(buf.data_ptr()), ws.value, ex, stream) == 0
    # the executor is gone: a second call must fail cleanly (two_phase_api.md: phase 2 may not be repeated)
    assert L.aclnnUpsampleNearest2d(ctypes.c_void_p(buf.data_ptr()), ws.value, ex, stream) == 161002
    torch.cuda.synchronize()
    assert torch.equal(y.cpu(), x.cpu().repeat_interleave(2, 2).repeat_interleave(2, 3))


@pytest.mark.parametrize("dtype", DTYPES)
def test_bicubic_aa_forward_bulk_copy_ring(ops, oracle, dev, dtype, monkeypatch):
    """The streaming forward kernel fed by bulk asynchronous copies into a shared-memory row ring (off by default,
    selected by OPSCV_AA_RING) gives the same result as the register-prefetch variant and the oracle."""
    x, x32 = quant(torch.rand((3, 2, 150, 96), generator=gen(60)), dtype)
    ref = oracle.bicubic_aa_fwd(x32, (33, 40), False)
    base = ops.upsample_bicubic2d_aa(x.to(dev), (33, 40), False)
    monkeypatch.setenv("OPSCV_AA_RING", "2")
    ring = ops.upsample_bicubic2d_aa(x.to(dev), (33, 40), False)
    monkeypatch.delenv("OPSCV_AA_RING")
    check(base, ref, dtype)
    check(ring, ref, dtype)
    assert torch.equal(base.view(torch.int32 if dtype == torch.float32 else torch.int16),
                       ring.view(torch.int32 if dtype == torch.float32 else torch.int16))
    assert ops.async_copy_timeouts() == 0


def test_no_device_wait_ran_out(ops, dev):
    """Collected after the operator tests of this file: none of the bounded waits on asynchronous copies gave up."""
    torch.cuda.synchronize(dev)
    assert ops.async_copy_timeouts() == 0


def _poison(t, rng, count):
    """Puts Inf / -Inf / NaN at `count` random positions plus the first and last element."""
    flat = t.reshape(-1)
    vals = [float("inf"), -float("inf"), float("nan")]
    idx = [0, flat.numel() - 1] + [int(i) for i in rng.integers(0, flat.numel(), count)]
    for j, i in enumerate(idx):
        flat[i] = vals[j % 3]
    return t


def _same_nonfinite(got, ref32, what):
    got = got.detach().cpu().float().numpy()
    assert np.array_equal(np.isnan(got), np.isnan(ref32)), what
    assert np.array_equal(np.isposinf(got), np.isposinf(ref32)), what
    assert np.array_equal(np.isneginf(got), np.isneginf(ref32)), what
    fin = np.isfinite(ref32)
    np.testing.assert_allclose(got[fin], ref32[fin], rtol=1e-5, atol=1e-5, err_msg=what)


@pytest.mark.parametrize("shape", [(2, 3, 8, 8, 16, 16), (1, 2, 8, 12, 16, 20), (2, 2, 9, 7, 5, 11), (1, 3, 40, 32, 9, 7)])
def test_nonfinite_values_spread_as_in_the_reference(ops, oracle, dev, shape):
    """An Inf or NaN in an input reaches exactly the outputs it reaches in the reference arithmetic: taps outside an
    output's window are never touched, zero-weight taps inside it are (0 * Inf = NaN). Covers the 2x kernels, the
    generic ones and the streaming bicubic-AA kernels (fp32)."""
    n, c, hi, wi, ho, wo = shape
    rng = np.random.default_rng(hi * 100 + wo)
    x = _poison(torch.randn((n, c, hi, wi), generator=gen(80)), rng, 3)
    go = _poison(torch.randn((n, c, ho, wo), generator=gen(81)), rng, 3)
    xd, god = x.to(dev), go.to(dev)
    _same_nonfinite(ops.upsample_nearest2d(xd, (ho, wo)), oracle.nearest2d_fwd(x.numpy(), (ho, wo)), "nearest fwd")
    _same_nonfinite(ops.upsample_nearest2d_backward(god, (ho, wo), (n, c, hi, wi)),
                    oracle.nearest2d_bwd(go.numpy(), (hi, wi)), "nearest bwd")
    for align in (False, True):
        _same_nonfinite(ops.upsample_bilinear2d(xd, (ho, wo), align), oracle.bilinear2d_fwd(x.numpy(), (ho, wo), align),
                        f"bilinear fwd align={align}")
        _same_nonfinite(ops.upsample_bilinear2d_backward(god, (ho, wo), (n, c, hi, wi), align),
                        oracle.bilinear2d_bwd(go.numpy(), (hi, wi), align), f"bilinear bwd align={align}")
    _same_nonfinite(ops.upsample_bicubic2d_aa(xd, (ho, wo), False), oracle.bicubic_aa_fwd(x.numpy(), (ho, wo), False),
                    "bicubic-AA fwd")
    _same_nonfinite(ops.upsample_bicubic2d_aa_grad(god, (ho, wo), (n, c, hi, wi), False),
                    oracle.bicubic_aa_bwd(go.numpy(), (hi, wi), False), "bicubic-AA bwd")


@pytest.mark.parametrize("shape", [(2, 8, 8, 8, 16, 16), (1, 5, 9, 7, 5, 11)])
def test_nonfinite_values_nhwc(ops, oracle, dev, shape):
    """The same check for the channels-last kernels (nearest and bilinear, both directions)."""
    n, c, hi, wi, ho, wo = shape
    rng = np.random.default_rng(hi * 10 + wo)
    x = _poison(torch.randn((n, hi, wi, c), generator=gen(82)), rng, 3)
    go = _poison(torch.randn((n, ho, wo, c), generator=gen(83)), rng, 3)
    xd, god = x.to(dev), go.to(dev)
    _same_nonfinite(ops.upsample_nearest2d(xd, (ho, wo), "NHWC"),
                    oracle.nearest2d_fwd(x.numpy(), (ho, wo), fmt=oracle.NHWC), "nearest fwd")
    _same_nonfinite(ops.upsample_nearest2d_backward(god, (ho, wo), (n, hi, wi, c), "NHWC"),
                    oracle.nearest2d_bwd(go.numpy(), (hi, wi), fmt=oracle.NHWC), "nearest bwd")
    for align in (False, True):
        _same_nonfinite(ops.upsample_bilinear2d(xd, (ho, wo), align, "NHWC"),
                        oracle.bilinear2d_fwd(x.numpy(), (ho, wo), align, fmt=oracle.NHWC), f"bilinear fwd {align}")
        _same_nonfinite(ops.upsample_bilinear2d_backward(god, (ho, wo), (n, hi, wi, c), align, "NHWC"),
                        oracle.bilinear2d_bwd(go.numpy(), (hi, wi), align, fmt=oracle.NHWC), f"bilinear bwd {align}")
