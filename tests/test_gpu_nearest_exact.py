"""GPU parity of UpsampleNearestExact2d / UpsampleNearestExact2dBackward, called through the C ABI, against the CPU
oracle on the same seeded inputs. The forward is a pure copy (exact in every dtype); the backward sums each window
in fp32 in row-major order like the oracle (exact in fp32, the rounded oracle value in fp16 / bf16)."""
import numpy as np
import pytest
import torch

from test_gpu_parity import DTYPES, SHAPES, check, gen, nhwc, quant

pytestmark = pytest.mark.gpu

EXTRA = [(1, 2, 33, 21, 7, 50), (2, 4, 12, 16, 36, 48), (1, 3, 10, 10, 10, 10), (1, 8, 16, 16, 64, 32)]


@pytest.mark.parametrize("sizes", [(64, 128), (56, 112), (7, 15), (16, 5), (1, 4), (5, 1), (1024, 224), (96, 288)])
def test_nearest_exact_tables_match_oracle_through_the_operator(ops, oracle, dev, sizes):
    """The index table is observable through the operator: an arange image comes back as the source indices."""
    i, o = sizes
    for scale in (0.0, 2.0, 1.7):
        x = torch.arange(i, dtype=torch.float32).reshape(1, 1, i, 1).to(dev)
        y = ops.upsample_nearest_exact2d(x, (o, 1), scales=(scale, 0.0))
        assert np.array_equal(y.cpu().numpy().reshape(-1).astype(np.int32), oracle.nearest_exact_src_index(i, o, scale))
        g = torch.zeros((1, 1, o, 1))
        s, e = oracle.nearest_exact_bwd_ranges(i, o, scale)
        g[0, 0, :, 0] = torch.arange(o, dtype=torch.float32) + 1.0
        gi = ops.upsample_nearest_exact2d_backward(g.to(dev), (o, 1), (1, 1, i, 1), scales=(scale, 0.0))
        want = np.array([np.arange(a, b, dtype=np.float64).sum() + (b - a) for a, b in zip(s, e)], dtype=np.float32)
        if o <= 2048:  # sums of small integers are exact in fp32
            assert np.array_equal(gi.cpu().numpy().reshape(-1), want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("fmt", ["NCHW", "NHWC"])
@pytest.mark.parametrize("shape", SHAPES + EXTRA)
def test_nearest_exact_forward(ops, oracle, dev, dtype, fmt, shape):
    n, c, hi, wi, ho, wo = shape
    x, x32 = quant(torch.randn((n, c, hi, wi), generator=gen(70)), dtype)
    xl = torch.from_numpy(nhwc(x32) if fmt == "NHWC" else x32).to(dtype)
    y = ops.upsample_nearest_exact2d(xl.to(dev), (ho, wo), fmt)
    ofmt = oracle.NHWC if fmt == "NHWC" else oracle.NCHW
    check(y, oracle.nearest_exact2d_fwd(nhwc(x32) if fmt == "NHWC" else x32, (ho, wo), fmt=ofmt), dtype, exact=True)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", SHAPES + EXTRA)
def test_nearest_exact_backward(ops, oracle, dev, dtype, shape):
    n, c, hi, wi, ho, wo = shape
    g, g32 = quant(torch.randn((n, c, ho, wo), generator=gen(71)), dtype)
    gi = ops.upsample_nearest_exact2d_backward(g.to(dev), (ho, wo), (n, c, hi, wi))
    check(gi, oracle.nearest_exact2d_bwd(g32, (hi, wi)), dtype, exact=True)


def test_nearest_exact_user_scales_and_torch(ops, oracle, dev):
    import torch.nn.functional as F
    x = torch.randn((2, 3, 9, 11), generator=gen(72))
    for scales in ((2.0, 2.0), (1.7, 2.3), (0.0, 1.5)):
        out = (18, 22)
        y = ops.upsample_nearest_exact2d(x.to(dev), out, scales=scales)
        assert np.array_equal(y.cpu().numpy(), oracle.nearest_exact2d_fwd(x.numpy(), out, scales))
        g = torch.randn((2, 3) + out, generator=gen(73))
        gi = ops.upsample_nearest_exact2d_backward(g.to(dev), out, (2, 3, 9, 11), scales=scales)
        assert np.array_equal(gi.cpu().numpy(), oracle.nearest_exact2d_bwd(g.numpy(), (9, 11), scales))
    # torch's CPU nearest-exact, an independent statement of the operator
    for shape, out in (((2, 3, 7, 9), (15, 20)), ((1, 2, 16, 12), (5, 7)), ((1, 1, 33, 21), (7, 50))):
        xt = torch.randn(shape, generator=gen(74)).requires_grad_(True)
        yt = F.interpolate(xt, size=out, mode="nearest-exact")
        gt = torch.randn(yt.shape, generator=gen(75))
        yt.backward(gt)
        assert torch.equal(ops.upsample_nearest_exact2d(xt.detach().to(dev), out).cpu(), yt.detach())
        got = ops.upsample_nearest_exact2d_backward(gt.to(dev), out, shape).cpu()
        np.testing.assert_allclose(got.numpy(), xt.grad.numpy(), rtol=1e-6, atol=1e-6)


def test_nearest_exact_strided_and_empty(ops, oracle, dev):
    base = torch.randn((2, 3, 12, 20), generator=gen(76)).to(dev)
    x = base[:, :, 1:10, 2:18:2]
    y = ops.upsample_nearest_exact2d(x, (20, 13))
    assert np.array_equal(y.cpu().numpy(), oracle.nearest_exact2d_fwd(x.contiguous().cpu().numpy(), (20, 13)))
    e = ops.upsample_nearest_exact2d(torch.zeros((0, 3, 4, 4), device=dev), (8, 8))
    assert e.shape == (0, 3, 8, 8)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("fmt", ["NCL", "ND"])
@pytest.mark.parametrize("lens", [(9, 20), (33, 7), (1, 5), (6, 1), (16, 32), (12, 12)])
def test_nearest_exact_1d(ops, oracle, dev, dtype, fmt, lens):
    """The 1-D pair is the 2-D operator on the (N, C, 1, L) view."""
    li, lo = lens
    x, x32 = quant(torch.randn((3, 4, li), generator=gen(77)), dtype)
    for scale in (0.0, 1.9):
        y = ops.upsample_nearest_exact1d(x.to(dev), lo, scale, fmt)
        ref = oracle.nearest_exact2d_fwd(x32.reshape(3, 4, 1, li), (1, lo), (1.0, scale)).reshape(3, 4, lo)
        check(y, ref, dtype, exact=True)
        g, g32 = quant(torch.randn((3, 4, lo), generator=gen(78)), dtype)
        gi = ops.upsample_nearest_exact1d_backward(g.to(dev), lo, (3, 4, li), scale, fmt)
        ref = oracle.nearest_exact2d_bwd(g32.reshape(3, 4, 1, lo), (1, li), (1.0, scale)).reshape(3, 4, li)
        check(gi, ref, dtype, exact=True)


def test_nearest_exact_1d_strided(ops, oracle, dev):
    base = torch.randn((2, 3, 40), generator=gen(79)).to(dev)
    x = base[:, :, 3:35:2]
    y = ops.upsample_nearest_exact1d(x, 37)
    ref = oracle.nearest_exact2d_fwd(x.contiguous().cpu().numpy().reshape(2, 3, 1, 16), (1, 37)).reshape(2, 3, 37)
    assert np.array_equal(y.cpu().numpy(), ref)
