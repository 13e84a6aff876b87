"""GPU parity of UpsampleNearest3d / UpsampleNearestExact3d, forward and backward, NCDHW and NDHWC, through the C ABI
against the CPU oracle: the forward is a copy (exact in every dtype), the backward sums each window in fp32 in the
oracle's order (exact in fp32, the rounded oracle value in 16-bit)."""
import numpy as np
import pytest
import torch

from test_gpu_parity import DTYPES, check, gen, quant

pytestmark = pytest.mark.gpu

SHAPES = [
    # (N, C, Din, Hin, Win, Dout, Hout, Wout)
    (2, 3, 4, 7, 9, 9, 15, 20),
    (1, 2, 8, 16, 12, 3, 5, 7),
    (1, 8, 4, 8, 8, 8, 16, 16),
    (1, 2, 1, 1, 1, 2, 4, 3),
    (1, 2, 4, 4, 3, 1, 1, 1),
    (2, 16, 3, 6, 8, 3, 12, 16),
    (1, 1, 5, 33, 40, 10, 17, 100),
]


def _cl(a):
    return np.ascontiguousarray(np.transpose(a, (0, 2, 3, 4, 1)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("fmt", ["NCDHW", "NDHWC"])
@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_nearest3d_forward_backward(ops, oracle, dev, dtype, fmt, exact, shape):
    n, c, di, hi, wi, do, ho, wo = shape
    ofmt = oracle.NHWC if fmt == "NDHWC" else oracle.NCHW
    x, x32 = quant(torch.randn((n, c, di, hi, wi), generator=gen(100)), dtype)
    xin = _cl(x32) if fmt == "NDHWC" else x32
    y = ops.upsample_nearest3d(torch.from_numpy(xin).to(dtype).to(dev), (do, ho, wo), fmt, exact=exact)
    check(y, oracle.nearest3d_fwd(xin, (do, ho, wo), exact=exact, fmt=ofmt), dtype, exact=True)
    g, g32 = quant(torch.randn((n, c, do, ho, wo), generator=gen(101)), dtype)
    gin = _cl(g32) if fmt == "NDHWC" else g32
    in_shape = (n, di, hi, wi, c) if fmt == "NDHWC" else (n, c, di, hi, wi)
    gi = ops.upsample_nearest3d_backward(torch.from_numpy(gin).to(dtype).to(dev), (do, ho, wo), in_shape, fmt, exact=exact)
    check(gi, oracle.nearest3d_bwd(gin, (di, hi, wi), exact=exact, fmt=ofmt), dtype, exact=True)


def test_nearest3d_user_scales_torch_and_views(ops, oracle, dev):
    import torch.nn.functional as F
    x = torch.randn((2, 3, 4, 6, 5), generator=gen(102))
    for exact, mode in ((False, "nearest"), (True, "nearest-exact")):
        xt = x.clone().requires_grad_(True)
        yt = F.interpolate(xt, size=(9, 13, 11), mode=mode)
        gt = torch.randn(yt.shape, generator=gen(103))
        yt.backward(gt)
        assert torch.equal(ops.upsample_nearest3d(x.to(dev), (9, 13, 11), exact=exact).cpu(), yt.detach())
        got = ops.upsample_nearest3d_backward(gt.to(dev), (9, 13, 11), tuple(x.shape), exact=exact).cpu()
        np.testing.assert_allclose(got.numpy(), xt.grad.numpy(), rtol=1e-6, atol=1e-6)
        scales = (2.0, 2.0, 2.0)
        y = ops.upsample_nearest3d(x.to(dev), (8, 12, 10), scales=scales, exact=exact)
        assert np.array_equal(y.cpu().numpy(), oracle.nearest3d_fwd(x.numpy(), (8, 12, 10), scales, exact=exact))
        g = torch.randn((2, 3, 8, 12, 10), generator=gen(104))
        gi = ops.upsample_nearest3d_backward(g.to(dev), (8, 12, 10), tuple(x.shape), scales=scales, exact=exact)
        assert np.array_equal(gi.cpu().numpy(), oracle.nearest3d_bwd(g.numpy(), (4, 6, 5), scales, exact=exact))
    # a strided 5-D view (cropped H and W: N and C merge, so four strided dimensions remain) and an empty batch
    base = torch.randn((2, 3, 4, 10, 12), generator=gen(105)).to(dev)
    view = base[:, :, :, 2:8, 1:11:2]
    y = ops.upsample_nearest3d(view, (8, 9, 7))
    assert np.array_equal(y.cpu().numpy(), oracle.nearest3d_fwd(view.contiguous().cpu().numpy(), (8, 9, 7)))
    e = ops.upsample_nearest3d(torch.zeros((0, 3, 4, 4, 4), device=dev), (8, 8, 8))
    assert e.shape == (0, 3, 8, 8, 8)
