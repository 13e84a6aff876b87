"""GPU parity of UpsampleBicubic2d / UpsampleBicubic2dBackward (cubic convolution, A = -0.75, no antialiasing),
called through the C ABI, against the CPU oracle on the same seeded inputs.

Bars:
  * forward, fp32: the oracle's bits (the kernel keeps the reference's operation order); fp16 / bf16: the fp32
    result rounded once, at most 1 ulp of the output dtype from the rounded oracle value;
  * backward, fp32: the bits of the oracle's statement of the reference's gather kernel (fixed summation order),
    and rtol 1e-5 / atol 1e-6 (plus the spread of the reference's own two kernels) against whichever kernel the
    reference's tiling selects for the arguments; 16-bit: 1 ulp under the same rule;
  * the copy schedules (equal extents, one pixel, integer positions): exact in every dtype.
"""
import numpy as np
import pytest
import torch

from test_gpu_parity import DTYPES, check, check_dispatched, gen, nhwc, quant

pytestmark = pytest.mark.gpu

SHAPES = [
    # (N, C, Hin, Win, Hout, Wout)
    (1, 3, 64, 64, 128, 128),   # 2x
    (2, 3, 7, 9, 15, 20),       # ragged up-scale
    (1, 4, 16, 24, 5, 7),       # down-scale
    (1, 2, 33, 17, 11, 40),     # down on H, up on W
    (1, 2, 1, 1, 3, 5),         # one input pixel
    (2, 2, 5, 6, 1, 1),         # one output pixel
    (1, 1, 3, 1, 7, 1),         # one column
    (1, 5, 9, 8, 9, 16),        # one axis unchanged
    (1, 2, 9, 9, 5, 5),         # align_corners: integer positions (scale 2)
    (1, 2, 15, 9, 5, 3),        # half pixel: odd integer scale 3 -> integer positions
    (1, 2, 8, 12, 4, 6),        # half pixel: even integer scale 2 -> general kernel
    (1, 16, 6, 8, 12, 16),      # wider channel count (NHWC)
    (1, 2, 2, 2, 9, 9),         # every grad_input element is a corner
    (1, 1, 3, 40, 8, 100),      # borders on H, long rows
]


def _layout(a, fmt):
    return nhwc(a) if fmt == "NHWC" else a


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("fmt", ["NCHW", "NHWC"])
@pytest.mark.parametrize("align", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_bicubic_forward(ops, oracle, dev, dtype, fmt, align, shape):
    n, c, hi, wi, ho, wo = shape
    x, x32 = quant(torch.randn((n, c, hi, wi), generator=gen(40)), dtype)
    xl = torch.from_numpy(_layout(x32, fmt)).to(dtype)
    y = ops.upsample_bicubic2d(xl.to(dev), (ho, wo), align, fmt)
    ofmt = oracle.NHWC if fmt == "NHWC" else oracle.NCHW
    ref = oracle.bicubic2d_fwd(_layout(x32, fmt), (ho, wo), align, fmt=ofmt)
    schedule = oracle.bicubic2d_fwd_schedule((hi, wi), (ho, wo), align)
    check(y, ref, dtype, exact=(dtype == torch.float32 or schedule != "general"))
    # the two layouts hold the same values
    assert np.array_equal(ref, _layout(oracle.bicubic2d_fwd(x32, (ho, wo), align), fmt))


def test_bicubic_forward_schedules(oracle):
    pick = oracle.bicubic2d_fwd_schedule
    assert pick((5, 5), (5, 5), False) == "copy"
    assert pick((5, 5), (5, 5), False, (1.7, 0.3)) == "copy"       # equal extents win over user scales
    assert pick((5, 6), (1, 1), True) == "one_output_pixel"
    assert pick((5, 6), (1, 1), False) == "general"
    assert pick((1, 1), (4, 3), False) == "one_input_pixel"
    assert pick((9, 9), (5, 5), True) == "integer_positions"
    assert pick((15, 9), (5, 3), False) == "integer_positions"
    assert pick((8, 12), (4, 6), False) == "general"
    assert pick((7, 9), (15, 20), True) == "general"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("fmt", ["NCHW", "NHWC"])
@pytest.mark.parametrize("align", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_bicubic_backward(ops, oracle, dev, dtype, fmt, align, shape):
    n, c, hi, wi, ho, wo = shape
    g, g32 = quant(torch.randn((n, c, ho, wo), generator=gen(41)), dtype)
    gl = torch.from_numpy(_layout(g32, fmt)).to(dtype)
    in_shape = (n, hi, wi, c) if fmt == "NHWC" else (n, c, hi, wi)
    gi = ops.upsample_bicubic2d_backward(gl.to(dev), (ho, wo), in_shape, align, fmt)
    gi2 = ops.upsample_bicubic2d_backward(gl.to(dev), (ho, wo), in_shape, align, fmt)
    assert torch.equal(gi, gi2)  # fixed summation order
    ofmt = oracle.NHWC if fmt == "NHWC" else oracle.NCHW
    gather = oracle.bicubic2d_bwd(_layout(g32, fmt), (hi, wi), align, fmt=ofmt, definition="gather")
    scatter = oracle.bicubic2d_bwd(_layout(g32, fmt), (hi, wi), align, fmt=ofmt, definition="scatter")
    check(gi, gather, dtype, exact=(dtype == torch.float32))
    choice = oracle.bicubic2d_bwd_kernel_choice((hi, wi), (ho, wo), align)
    if choice == "scatter":
        check_dispatched(gi, scatter, gather, dtype)
    # the deterministic option selects the gather kernel in the reference; here it changes nothing
    ops.set_deterministic(True)
    try:
        gd = ops.upsample_bicubic2d_backward(gl.to(dev), (ho, wo), in_shape, align, fmt)
    finally:
        ops.set_deterministic(False)
    assert torch.equal(gd, gi)


def test_bicubic_backward_kernel_choice(oracle):
    pick = oracle.bicubic2d_bwd_kernel_choice
    assert pick((8, 8), (8, 8), False) == "copy"
    assert pick((8, 8), (16, 16), False) == "gather"                       # an extent grows
    assert pick((16, 16), (5, 7), False) == "scatter"                      # down-scale, no fixed order asked
    assert pick((16, 16), (5, 7), False, deterministic=True) == "gather"
    assert pick((16, 16), (5, 7), False, scales=(2.0, 0.0)) == "gather"    # a user scale puts the ratio in (0, 1)
    assert pick((16, 8), (5, 8), True) == "scatter"


def test_bicubic_user_scales(ops, oracle, dev):
    x = torch.randn((1, 2, 8, 10), generator=gen(42))
    for scales in ((2.0, 2.0), (2.4, 1.9), (0.0, 3.0)):
        y = ops.upsample_bicubic2d(x.to(dev), (19, 21), False, scales=scales)
        check(y, oracle.bicubic2d_fwd(x.numpy(), (19, 21), False, scales), torch.float32, exact=True)
        g = torch.randn((1, 2, 19, 21), generator=gen(43))
        gi = ops.upsample_bicubic2d_backward(g.to(dev), (19, 21), (1, 2, 8, 10), False, scales=scales)
        check(gi, oracle.bicubic2d_bwd(g.numpy(), (8, 10), False, scales, definition="gather"), torch.float32,
              exact=True)
        check(gi, oracle.bicubic2d_bwd(g.numpy(), (8, 10), False, scales, definition="scatter"), torch.float32)
    # align_corners ignores user scales
    y = ops.upsample_bicubic2d(x.to(dev), (19, 21), True, scales=(5.0, 7.0))
    check(y, oracle.bicubic2d_fwd(x.numpy(), (19, 21), True), torch.float32, exact=True)


def test_bicubic_matches_torch_cpu(ops, dev):
    """An independent statement of the operator: torch's CPU bicubic (same coefficient A = -0.75) in float64."""
    import torch.nn.functional as F
    for shape, out, align in (((2, 3, 7, 9), (15, 20), False), ((1, 2, 16, 12), (5, 7), True),
                              ((1, 1, 5, 5), (15, 15), False)):
        x = torch.randn(shape, generator=gen(44), dtype=torch.float64).requires_grad_(True)
        y = F.interpolate(x, size=out, mode="bicubic", align_corners=align)
        g = torch.randn(y.shape, generator=gen(45), dtype=torch.float64)
        y.backward(g)
        got = ops.upsample_bicubic2d(x.detach().float().to(dev), out, align)
        np.testing.assert_allclose(got.cpu().numpy(), y.detach().float().numpy(), rtol=1e-5, atol=1e-5)
        gi = ops.upsample_bicubic2d_backward(g.float().to(dev), out, shape, align)
        np.testing.assert_allclose(gi.cpu().numpy(), x.grad.float().numpy(), rtol=1e-5, atol=1e-5)


def test_bicubic_strided_views_and_empty(ops, oracle, dev):
    base = torch.randn((2, 3, 12, 20), generator=gen(46)).to(dev)
    x = base[:, :, 1:10, 2:18:2]                      # strided input view
    out_base = torch.zeros((2, 3, 20, 40), device=dev)
    out = out_base[:, :, :, ::2]                      # strided output view
    ops.upsample_bicubic2d(x, (20, 20), False, out=out)
    ref = oracle.bicubic2d_fwd(x.contiguous().cpu().numpy(), (20, 20), False)
    assert np.array_equal(out.cpu().numpy(), ref)
    assert float(out_base[:, :, :, 1::2].abs().max()) == 0.0
    e = ops.upsample_bicubic2d(torch.zeros((0, 3, 4, 4), device=dev), (8, 8))
    assert e.shape == (0, 3, 8, 8)
    e = ops.upsample_bicubic2d_backward(torch.zeros((0, 3, 8, 8), device=dev), (8, 8), (0, 3, 4, 4))
    assert e.shape == (0, 3, 4, 4)


def test_bicubic_non_finite_values(ops, oracle, dev):
    """Same-size calls copy (an Inf stays an Inf); in the general kernel an Inf reaches the outputs whose sixteen
    taps include it, exactly as in the oracle."""
    x = torch.randn((1, 2, 6, 7), generator=gen(47))
    x[0, 0, 2, 3] = float("inf")
    x[0, 1, 5, 6] = float("nan")
    same = ops.upsample_bicubic2d(x.to(dev), (6, 7), False)
    assert torch.equal(same.cpu().nan_to_num(7.0, 8.0, 9.0), x.nan_to_num(7.0, 8.0, 9.0))
    y = ops.upsample_bicubic2d(x.to(dev), (13, 15), False).cpu().numpy()
    ref = oracle.bicubic2d_fwd(x.numpy(), (13, 15), False)
    assert np.array_equal(np.isnan(y), np.isnan(ref)) and np.array_equal(np.isinf(y), np.isinf(ref))
    fin = np.isfinite(ref)
    assert np.array_equal(y[fin], ref[fin])


def test_bicubic_larger_case_is_bit_exact(ops, oracle, dev):
    """A case with more rows than the launch grid has row blocks, so the row loop of both kernels wraps."""
    x = torch.randn((40, 8, 24, 24), generator=gen(48))
    y = ops.upsample_bicubic2d(x.to(dev), (48, 48), False)
    assert np.array_equal(y.cpu().numpy(), oracle.bicubic2d_fwd(x.numpy(), (48, 48), False))
    g = torch.randn((40, 8, 48, 48), generator=gen(49))
    gi = ops.upsample_bicubic2d_backward(g.to(dev), (48, 48), (40, 8, 24, 24), False)
    assert np.array_equal(gi.cpu().numpy(), oracle.bicubic2d_bwd(g.numpy(), (24, 24), False, definition="gather"))


X2_SHAPES = [
    # (N, C, Hin, Win): grad_output is (N, C, 2 Hin, 2 Win)
    (1, 2, 2, 2),      # corners only
    (2, 1, 2, 5),      # two rows, both borders; odd width
    (1, 3, 3, 3),      # one interior element
    (1, 2, 5, 4),      # wout a multiple of 8: 16-byte staging loads for fp16
    (2, 2, 7, 13),     # odd width: the last pair holds one column
    (1, 1, 4, 300),    # a row longer than a block
    (3, 2, 61, 20),    # several bands per plane, the last one short
    (1, 1, 9, 1100),   # a wide row: one band row per block
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", X2_SHAPES)
def test_bicubic_backward_at_2x(ops, oracle, dev, dtype, shape):
    """The staged 2x kernel (NCHW, align_corners = false, scales 0.5): the oracle's bits in fp32, every border kind."""
    n, c, hi, wi = shape
    g, g32 = quant(torch.randn((n, c, 2 * hi, 2 * wi), generator=gen(140)), dtype)
    gi = ops.upsample_bicubic2d_backward(g.to(dev), (2 * hi, 2 * wi), (n, c, hi, wi), False)
    ref = oracle.bicubic2d_bwd(g32, (hi, wi), False, definition="gather")
    check(gi, ref, dtype, exact=(dtype == torch.float32))
    # a view with an offset base (the staging loads fall back to single elements when the base is not 16-byte aligned)
    flat = torch.zeros(g.numel() + 1, dtype=dtype)
    flat[1:] = g.flatten()
    gv = flat.to(dev)[1:].view(n, c, 2 * hi, 2 * wi)
    assert torch.equal(ops.upsample_bicubic2d_backward(gv, (2 * hi, 2 * wi), (n, c, hi, wi), False), gi)


def test_bicubic_backward_at_2x_special_values(ops, oracle, dev):
    """Inf / NaN grads reach exactly the grad_input elements whose walk includes them (the zero columns beside a
    staged row never meet them), and sums of signed zeros keep the oracle's sign."""
    g = torch.randn((1, 2, 12, 16), generator=gen(141))
    g[0, 0, 0, 0] = float("inf")
    g[0, 0, 11, 15] = float("-inf")
    g[0, 1, 5, 7] = float("nan")
    g[0, 1, 0, 15] = float("inf")
    gi = ops.upsample_bicubic2d_backward(g.to(dev), (12, 16), (1, 2, 6, 8), False).cpu().numpy()
    ref = oracle.bicubic2d_bwd(g.numpy(), (6, 8), False, definition="gather")
    assert np.array_equal(np.isnan(gi), np.isnan(ref)) and np.array_equal(np.isinf(gi), np.isinf(ref))
    fin = np.isfinite(ref)
    assert np.array_equal(gi[fin], ref[fin])
    z = torch.zeros((1, 1, 8, 8))
    z[0, 0, :, ::2] = -0.0
    z[0, 0, 3, 3] = -1e-45  # a denormal whose products underflow to -0
    gz = ops.upsample_bicubic2d_backward(z.to(dev), (8, 8), (1, 1, 4, 4), False).cpu().numpy()
    rz = oracle.bicubic2d_bwd(z.numpy(), (4, 4), False, definition="gather")
    assert np.array_equal(gz.view(np.uint32), rz.view(np.uint32))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", X2_SHAPES + [(1, 2, 1, 2), (2, 3, 1, 8), (1, 1, 70, 64), (2, 2, 33, 6), (1, 2, 3, 1), (2, 1, 5, 21), (1, 3, 13, 25)])
def test_bicubic_forward_at_2x(ops, oracle, dev, dtype, shape):
    """The staged 2x forward (NCHW, half-pixel; odd input widths leave the last group of four columns half used): the
    oracle's bits in fp32, borders by replicated rows and columns."""
    n, c, hi, wi = shape
    x, x32 = quant(torch.randn((n, c, hi, wi), generator=gen(142)), dtype)
    y = ops.upsample_bicubic2d(x.to(dev), (2 * hi, 2 * wi), False)
    check(y, oracle.bicubic2d_fwd(x32, (2 * hi, 2 * wi), False), dtype, exact=(dtype == torch.float32))
    flat = torch.zeros(x.numel() + 1, dtype=dtype)
    flat[1:] = x.flatten()
    xv = flat.to(dev)[1:].view(n, c, hi, wi)  # a base that is not 16-byte aligned: single-element staging loads
    assert torch.equal(ops.upsample_bicubic2d(xv, (2 * hi, 2 * wi), False), y)
    xs = torch.randn((n, c, hi, wi), generator=gen(143))
    xs[0, 0, 0, 0] = float("inf")
    xs[-1, -1, -1, -1] = float("nan")
    ys = ops.upsample_bicubic2d(xs.to(dev), (2 * hi, 2 * wi), False).cpu().numpy()
    ref = oracle.bicubic2d_fwd(xs.numpy(), (2 * hi, 2 * wi), False)
    assert np.array_equal(np.isnan(ys), np.isnan(ref)) and np.array_equal(np.isinf(ys), np.isinf(ref))
    fin = np.isfinite(ref)
    assert np.array_equal(ys[fin], ref[fin])


def test_bicubic_2x_random_extents(ops, oracle, dev):
    """Random extents at exactly 2x through both staged kernels (fp32: the oracle's bits): band counts, short last
    bands, odd and even widths, widths past one block, the fall-back to the general kernels for very wide rows."""
    rng = np.random.default_rng(20260)
    shapes = [(int(rng.integers(1, 3)), int(rng.integers(1, 4)), int(rng.integers(1, 90)), int(rng.integers(1, 200)))
              for _ in range(24)] + [(1, 1, 3, 800), (1, 1, 130, 7), (1, 2, 95, 96)]
    for i, (n, c, hi, wi) in enumerate(shapes):
        x = torch.randn((n, c, hi, wi), generator=gen(300 + i))
        g = torch.randn((n, c, 2 * hi, 2 * wi), generator=gen(400 + i))
        y = ops.upsample_bicubic2d(x.to(dev), (2 * hi, 2 * wi), False)
        assert np.array_equal(y.cpu().numpy(), oracle.bicubic2d_fwd(x.numpy(), (2 * hi, 2 * wi), False)), (n, c, hi, wi)
        gi = ops.upsample_bicubic2d_backward(g.to(dev), (2 * hi, 2 * wi), (n, c, hi, wi), False)
        assert np.array_equal(gi.cpu().numpy(),
                              oracle.bicubic2d_bwd(g.numpy(), (hi, wi), False, definition="gather")), (n, c, hi, wi)
