"""GPU parity of UpsampleBilinear2dAA / UpsampleBilinear2dAABackward (anti-aliased resampling with a triangle
filter, NCHW), called through the C ABI, against the CPU oracle on the same seeded inputs.

Bars: window starts and sizes bit-exact, normalised fp32 weights bit for bit; forward and backward values rtol 1e-5 /
atol 1e-6 in fp32 (the kernels keep the oracle's terms but tile the sums), at most 1 ulp of the output dtype for
fp16 / bf16; the deterministic option gives the same bits on every run."""
import numpy as np
import pytest
import torch

from test_gpu_parity import AA_SHAPES, DTYPES, check, check_dispatched, gen, quant

pytestmark = pytest.mark.gpu

SHAPES = AA_SHAPES + [(2, 2, 48, 64, 12, 16), (1, 3, 17, 19, 40, 33), (1, 2, 30, 8, 7, 8)]


@pytest.mark.parametrize("sizes", [(64, 128), (56, 14), (7, 15), (16, 5), (1, 4), (5, 1), (1024, 224), (96, 96)])
def test_bilinear_aa_tables_bit_exact(ops, oracle, sizes):
    i, o = sizes
    for scale in (0.0, 2.0, 0.3):
        for align in (False, True):
            xmin, xsize, w = ops.debug_axis_table("bilinear_aa", i, o, align, scale)
            rmin, rsize, rw = oracle.bilinear_aa_table(i, o, align, scale)
            assert np.array_equal(xmin, rmin) and np.array_equal(xsize, rsize)
            assert w.shape[1] >= rw.shape[1]
            assert np.array_equal(w[:, :rw.shape[1]].view(np.int32), rw.view(np.int32))
            assert not w[:, rw.shape[1]:].any()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("align", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_bilinear_aa_forward(ops, oracle, dev, dtype, align, shape):
    n, c, hi, wi, ho, wo = shape
    x, x32 = quant(torch.rand((n, c, hi, wi), generator=gen(60)), dtype)
    y = ops.upsample_bilinear2d_aa(x.to(dev), (ho, wo), align)
    check(y, oracle.bilinear_aa_fwd(x32, (ho, wo), align), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("align", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("algo", ["gather", "atomic"])
def test_bilinear_aa_backward(ops, oracle, dev, dtype, align, shape, algo):
    n, c, hi, wi, ho, wo = shape
    g, g32 = quant(torch.randn((n, c, ho, wo), generator=gen(61)), dtype)
    ops.set_backward_algo(algo)
    try:
        gi = ops.upsample_bilinear2d_aa_backward(g.to(dev), (ho, wo), (n, c, hi, wi), align)
    finally:
        ops.set_backward_algo("gather")
    scatter = oracle.bilinear_aa_bwd(g32, (hi, wi), align, definition="scatter")
    gather = oracle.bilinear_aa_bwd(g32, (hi, wi), align, definition="gather")
    # the reference's two kernels add the same terms; a 16-bit result that cancels to nearly zero is held to the
    # absolute bar (its ulp is far below the rounding of the fp32 sum)
    if dtype == torch.float32:
        check(gi, scatter, dtype)
        check(gi, gather, dtype)
    else:
        check_dispatched(gi, scatter, gather, dtype)
    ops.set_deterministic(True)
    try:
        gd = ops.upsample_bilinear2d_aa_backward(g.to(dev), (ho, wo), (n, c, hi, wi), align)
        gd2 = ops.upsample_bilinear2d_aa_backward(g.to(dev), (ho, wo), (n, c, hi, wi), align)
    finally:
        ops.set_deterministic(False)
    assert torch.equal(gd, gd2)
    if dtype == torch.float32:
        check(gd, gather, dtype)
    else:
        check_dispatched(gd, gather, scatter, dtype)


def test_bilinear_aa_user_scales_and_copy(ops, oracle, dev):
    x = torch.rand((1, 2, 20, 24), generator=gen(62))
    for scales in ((0.5, 1.0 / 3.0), (0.45, 0.3), (0.0, 0.5)):
        y = ops.upsample_bilinear2d_aa(x.to(dev), (10, 8), False, scales=scales)
        check(y, oracle.bilinear_aa_fwd(x.numpy(), (10, 8), False, scales), torch.float32)
        g = torch.randn((1, 2, 10, 8), generator=gen(63))
        gi = ops.upsample_bilinear2d_aa_backward(g.to(dev), (10, 8), (1, 2, 20, 24), False, scales=scales)
        check(gi, oracle.bilinear_aa_bwd(g.numpy(), (20, 24), False, scales), torch.float32)
    # equal extents with a scale of one copy the tensor (an Inf stays an Inf)
    x[0, 0, 3, 4] = float("inf")
    same = ops.upsample_bilinear2d_aa(x.to(dev), (20, 24), False)
    assert torch.equal(same.cpu(), x)
    back = ops.upsample_bilinear2d_aa_backward(x.to(dev), (20, 24), (1, 2, 20, 24), False)
    assert torch.equal(back.cpu(), x)


def test_bilinear_aa_matches_torch_cpu(ops, dev):
    """An independent statement of the operator: torch's CPU anti-aliased bilinear in float64."""
    import torch.nn.functional as F
    for shape, out, align in (((2, 3, 32, 40), (7, 9), False), ((1, 2, 6, 7), (13, 15), True),
                              ((1, 1, 64, 64), (14, 14), False)):
        x = torch.randn(shape, generator=gen(64), dtype=torch.float64).requires_grad_(True)
        y = F.interpolate(x, size=out, mode="bilinear", align_corners=align, antialias=True)
        g = torch.randn(y.shape, generator=gen(65), dtype=torch.float64)
        y.backward(g)
        got = ops.upsample_bilinear2d_aa(x.detach().float().to(dev), out, align)
        np.testing.assert_allclose(got.cpu().numpy(), y.detach().float().numpy(), rtol=1e-5, atol=2e-6)
        gi = ops.upsample_bilinear2d_aa_backward(g.float().to(dev), out, shape, align)
        np.testing.assert_allclose(gi.cpu().numpy(), x.grad.float().numpy(), rtol=1e-5, atol=2e-6)


def test_bilinear_aa_strided_and_empty(ops, oracle, dev):
    base = torch.rand((2, 3, 40, 50), generator=gen(66)).to(dev)
    x = base[:, :, 4:36, 1:49:2]
    y = ops.upsample_bilinear2d_aa(x, (9, 11), False)
    check(y, oracle.bilinear_aa_fwd(x.contiguous().cpu().numpy(), (9, 11), False), torch.float32)
    e = ops.upsample_bilinear2d_aa(torch.zeros((0, 3, 8, 8), device=dev), (4, 4))
    assert e.shape == (0, 3, 4, 4)
