"""GPU parity of UpsampleTrilinear3d / UpsampleTrilinear3dBackward, NCDHW and NDHWC, through the C ABI against the
CPU oracle.

Bars:
  * forward, fp32: the oracle's bits (the kernel keeps the operation order of the reference's SIMT loops, the fused
    multiply-adds of its coordinate and of its one-axis loops included); fp16 / bf16: the fp32 value rounded once, at
    most 1 ulp of the output dtype from the rounded oracle value; copies are exact;
  * backward: the reference computes three separable matrix products (W, H, D) in fp32, whose internal summation
    order is the matrix unit's; the oracle and the kernel both take ascending grad_output order in each stage, so
    they agree bit for bit in fp32, and the bar against the reference itself is rtol 1e-5 / atol 1e-6 (checked here
    against torch in float64); 16-bit: the fp32 value rounded once, 1 ulp.
"""
import numpy as np
import pytest
import torch

from test_gpu_parity import DTYPES, check, gen, quant

pytestmark = pytest.mark.gpu

SHAPES = [
    # (N, C, Din, Hin, Win, Dout, Hout, Wout)
    (2, 3, 4, 7, 9, 9, 15, 20),      # ragged up-scale on every axis
    (1, 2, 8, 16, 12, 3, 5, 7),      # down-scale
    (1, 8, 4, 8, 8, 8, 16, 16),      # 2x
    (1, 2, 1, 1, 1, 2, 4, 3),        # one input voxel
    (1, 2, 4, 4, 3, 1, 1, 1),        # one output voxel
    (2, 16, 3, 6, 8, 3, 12, 16),     # D unchanged
    (1, 2, 5, 6, 7, 10, 6, 7),       # only D resampled (two-tap loop)
    (1, 2, 5, 6, 7, 5, 9, 7),        # only H resampled
    (1, 4, 5, 6, 7, 5, 6, 20),       # only W resampled
    (1, 3, 4, 5, 6, 4, 5, 6),        # equal extents: a copy
    (1, 1, 5, 33, 40, 10, 17, 100),  # long rows
]


def _cl(a):
    return np.ascontiguousarray(np.transpose(a, (0, 2, 3, 4, 1)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("fmt", ["NCDHW", "NDHWC"])
@pytest.mark.parametrize("align", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_trilinear3d_forward_backward(ops, oracle, dev, dtype, fmt, align, shape):
    n, c, di, hi, wi, do, ho, wo = shape
    ofmt = oracle.NHWC if fmt == "NDHWC" else oracle.NCHW
    x, x32 = quant(torch.randn((n, c, di, hi, wi), generator=gen(110)), dtype)
    xin = _cl(x32) if fmt == "NDHWC" else x32
    y = ops.upsample_trilinear3d(torch.from_numpy(xin).to(dtype).to(dev), (do, ho, wo), align, fmt)
    loop = oracle.trilinear3d_fwd_loop((di, hi, wi), (do, ho, wo), align)
    check(y, oracle.trilinear3d_fwd(xin, (do, ho, wo), align, fmt=ofmt), dtype,
          exact=(dtype == torch.float32 or loop == "copy"))
    g, g32 = quant(torch.randn((n, c, do, ho, wo), generator=gen(111)), dtype)
    gin = _cl(g32) if fmt == "NDHWC" else g32
    gi = ops.upsample_trilinear3d_backward(torch.from_numpy(gin).to(dtype).to(dev), (do, ho, wo), (n, c, di, hi, wi),
                                           align, fmt)
    gi2 = ops.upsample_trilinear3d_backward(torch.from_numpy(gin).to(dtype).to(dev), (do, ho, wo), (n, c, di, hi, wi),
                                            align, fmt)
    assert torch.equal(gi, gi2)  # fixed summation order
    check(gi, oracle.trilinear3d_bwd(gin, (di, hi, wi), align, fmt=ofmt), dtype, exact=(dtype == torch.float32))


def test_trilinear3d_loops(oracle):
    pick = oracle.trilinear3d_fwd_loop
    assert pick((4, 5, 6), (4, 5, 6), False) == "copy"
    assert pick((4, 5, 6), (4, 5, 6), False, (1.7, 0.3, 2.0)) == "copy"   # equal extents win over user scales
    assert pick((4, 5, 6), (8, 5, 6), False) == "d_only"
    assert pick((4, 5, 6), (4, 9, 6), True) == "h_only"
    assert pick((4, 5, 6), (4, 5, 3), False) == "w_only"
    assert pick((4, 5, 6), (8, 10, 6), False) == "full"
    assert pick((4, 5, 6), (8, 10, 12), True) == "full"
    assert oracle.trilinear3d_scale(4, 8, False, (0, 0, 0), 0) == 0.5
    assert oracle.trilinear3d_scale(4, 9, False, (2.25, 2.0, 2.0), 0) == np.float32(1.0 / 2.25)
    assert oracle.trilinear3d_scale(4, 9, False, (2.25, 0.0, 2.0), 0) == np.float32(4.0 / 9.0)  # one scale missing
    assert oracle.trilinear3d_scale(4, 9, True, (2.25, 2.0, 2.0), 0) == np.float32(3.0) / np.float32(8.0)
    assert oracle.trilinear3d_scale(4, 1, True, (0, 0, 0), 0) == 0.0


def test_trilinear3d_user_scales_and_torch(ops, oracle, dev):
    import torch.nn.functional as F
    x = torch.randn((2, 3, 4, 6, 5), generator=gen(112))
    for align in (False, True):
        xt = x.double().requires_grad_(True)
        yt = F.interpolate(xt, size=(9, 13, 11), mode="trilinear", align_corners=align)
        gt = torch.randn(yt.shape, generator=gen(113), dtype=torch.float64)
        yt.backward(gt)
        y = ops.upsample_trilinear3d(x.to(dev), (9, 13, 11), align)
        np.testing.assert_allclose(y.cpu().numpy(), yt.detach().float().numpy(), rtol=1e-5, atol=1e-5)
        gi = ops.upsample_trilinear3d_backward(gt.float().to(dev), (9, 13, 11), tuple(x.shape), align)
        np.testing.assert_allclose(gi.cpu().numpy(), xt.grad.float().numpy(), rtol=1e-5, atol=1e-5)
    for scales in ((2.25, 2.2, 2.3), (2.25, 0.0, 2.3)):
        y = ops.upsample_trilinear3d(x.to(dev), (9, 13, 11), False, scales=scales)
        assert np.array_equal(y.cpu().numpy(), oracle.trilinear3d_fwd(x.numpy(), (9, 13, 11), False, scales))
        g = torch.randn((2, 3, 9, 13, 11), generator=gen(114))
        gi = ops.upsample_trilinear3d_backward(g.to(dev), (9, 13, 11), tuple(x.shape), False, scales=scales)
        assert np.array_equal(gi.cpu().numpy(), oracle.trilinear3d_bwd(g.numpy(), (4, 6, 5), False, scales))
    # align_corners ignores the user scales
    y = ops.upsample_trilinear3d(x.to(dev), (9, 13, 11), True, scales=(5.0, 7.0, 3.0))
    assert np.array_equal(y.cpu().numpy(), oracle.trilinear3d_fwd(x.numpy(), (9, 13, 11), True))


def test_trilinear3d_views_and_empty(ops, oracle, dev):
    # a strided 5-D view (cropped H and W: N and C merge, so four strided dimensions remain) and an empty batch
    base = torch.randn((2, 3, 4, 10, 12), generator=gen(115)).to(dev)
    view = base[:, :, :, 2:8, 1:11:2]
    y = ops.upsample_trilinear3d(view, (8, 9, 7))
    assert np.array_equal(y.cpu().numpy(), oracle.trilinear3d_fwd(view.contiguous().cpu().numpy(), (8, 9, 7)))
    gbase = torch.randn((2, 3, 8, 9, 14), generator=gen(116)).to(dev)
    gview = gbase[..., ::2]
    gi = ops.upsample_trilinear3d_backward(gview, (8, 9, 7), (2, 3, 4, 6, 5))
    assert np.array_equal(gi.cpu().numpy(), oracle.trilinear3d_bwd(gview.contiguous().cpu().numpy(), (4, 6, 5)))
    e = ops.upsample_trilinear3d(torch.zeros((0, 3, 4, 4, 4), device=dev), (8, 8, 8))
    assert e.shape == (0, 3, 8, 8, 8)
    e = ops.upsample_trilinear3d_backward(torch.zeros((0, 3, 8, 8, 8), device=dev), (8, 8, 8), (0, 3, 4, 4, 4))
    assert e.shape == (0, 3, 4, 4, 4)


def test_trilinear3d_non_finite_values(ops, oracle, dev):
    """A tap that holds Inf or NaN under a zero weight makes the output NaN (the plain product 0 * Inf would as
    well; the reference tests it explicitly), and the one-axis loops turn every Inf / NaN tap into NaN."""
    x = torch.randn((1, 2, 4, 5, 6), generator=gen(117))
    x[0, 0, 1, 2, 3] = float("inf")
    x[0, 1, 3, 4, 5] = float("nan")
    x[0, 1, 0, 0, 0] = float("-inf")
    for out, align in (((8, 10, 12), False), ((7, 9, 11), True), ((8, 5, 6), False), ((4, 5, 12), True)):
        y = ops.upsample_trilinear3d(x.to(dev), out, align).cpu().numpy()
        ref = oracle.trilinear3d_fwd(x.numpy(), out, align)
        assert np.array_equal(np.isnan(y), np.isnan(ref)) and np.array_equal(np.isinf(y), np.isinf(ref))
        fin = np.isfinite(ref)
        assert np.array_equal(y[fin], ref[fin])
    same = ops.upsample_trilinear3d(x.to(dev), (4, 5, 6), False)
    assert torch.equal(same.cpu().nan_to_num(7.0, 8.0, 9.0), x.nan_to_num(7.0, 8.0, 9.0))


def test_trilinear3d_larger_case_is_bit_exact(ops, oracle, dev):
    """More rows than the launch grid has row blocks, so the row loop of both kernels wraps."""
    x = torch.randn((6, 8, 12, 24, 24), generator=gen(118))
    y = ops.upsample_trilinear3d(x.to(dev), (24, 48, 48), False)
    assert np.array_equal(y.cpu().numpy(), oracle.trilinear3d_fwd(x.numpy(), (24, 48, 48), False))
    g = torch.randn((6, 8, 24, 48, 48), generator=gen(119))
    gi = ops.upsample_trilinear3d_backward(g.to(dev), (24, 48, 48), (6, 8, 12, 24, 24), False)
    assert np.array_equal(gi.cpu().numpy(), oracle.trilinear3d_bwd(g.numpy(), (12, 24, 24), False))
