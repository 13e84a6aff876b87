"""GPU parity of GridSampler3D / GridSampler3DBackward through the C ABI against the CPU oracle: the forward keeps
the reference's tap and operation order (fp32: the oracle's bits, 16-bit: 1 ulp); grad_grid is one thread's ordered
sum (fp32 bits of the oracle), grad_input is an atomic sum (rtol 1e-5 / atol 1e-6 with the absolute term scaled by the
largest magnitude, as for the 2-D atomic backward)."""
import numpy as np
import pytest
import torch

from test_gpu_parity import DTYPES, check, gen, quant

pytestmark = pytest.mark.gpu


def make_grid(n, do, ho, wo, seed, span=1.2):
    return torch.rand((n, do, ho, wo, 3), generator=gen(seed)) * 2 * span - span


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pad", [0, 1, 2])
@pytest.mark.parametrize("align", [False, True])
def test_grid_sampler3d_forward(ops, oracle, dev, dtype, pad, align):
    x, x32 = quant(torch.randn((2, 5, 6, 7, 9), generator=gen(110)), dtype)
    grid, g32 = quant(make_grid(2, 4, 5, 6, 111), dtype)
    y = ops.grid_sampler3d(x.to(dev), grid.to(dev), 0, pad, align)
    check(y, oracle.grid_sampler3d_fwd(x32, g32, pad, align), dtype, exact=(dtype == torch.float32))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("interp", [0, 1])
@pytest.mark.parametrize("pad", [0, 1, 2])
@pytest.mark.parametrize("align", [False, True])
def test_grid_sampler3d_backward(ops, oracle, dev, dtype, interp, pad, align):
    x, x32 = quant(torch.randn((2, 5, 6, 7, 9), generator=gen(112)), dtype)
    grid, g32 = quant(make_grid(2, 4, 5, 6, 113), dtype)
    go, go32 = quant(torch.randn((2, 5, 4, 5, 6), generator=gen(114)), dtype)
    gi, gg = ops.grid_sampler3d_backward(go.to(dev), x.to(dev), grid.to(dev), interp, pad, align)
    ri, rg = oracle.grid_sampler3d_bwd(go32, x32, g32, interp, pad, align)
    if dtype == torch.float32:
        np.testing.assert_allclose(gi.cpu().numpy(), ri, rtol=1e-5, atol=1e-6 * max(1.0, float(np.abs(ri).max())))
        assert np.array_equal(gg.cpu().numpy(), rg)
    else:
        check(gg, rg, dtype)
        want = torch.from_numpy(ri).to(dtype).float().numpy()
        step = np.maximum(np.abs(want) * (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10), 1e-6 * max(1.0, float(np.abs(ri).max())))
        assert (np.abs(gi.float().cpu().numpy() - ri) <= step * 1.01 + 1e-6).all()
    # masks: an output that is not wanted is left untouched
    keep_i, keep_g = torch.full_like(x, 7.0).to(dev), torch.full_like(grid, 7.0).to(dev)
    ops.grid_sampler3d_backward(go.to(dev), x.to(dev), grid.to(dev), interp, pad, align, mask=(True, False),
                                input_grad=keep_i, grid_grad=keep_g)
    assert torch.equal(keep_g.cpu(), torch.full_like(grid, 7.0)) and not torch.equal(keep_i.cpu(), torch.full_like(x, 7.0))


def test_grid_sampler3d_torch_nearest_layouts_and_special_values(ops, oracle, dev):
    import torch.nn.functional as F
    x = torch.randn((2, 3, 5, 6, 7), generator=gen(115), dtype=torch.float64)
    grid = make_grid(2, 4, 5, 6, 116).double()
    for pad, name in enumerate(("zeros", "border", "reflection")):
        for align in (False, True):
            xt, gt = x.clone().requires_grad_(True), grid.clone().requires_grad_(True)
            yt = F.grid_sample(xt, gt, mode="bilinear", padding_mode=name, align_corners=align)
            g = torch.randn(yt.shape, generator=gen(117), dtype=torch.float64)
            yt.backward(g)
            y = ops.grid_sampler3d(x.float().to(dev), grid.float().to(dev), 0, pad, align)
            np.testing.assert_allclose(y.cpu().numpy(), yt.detach().float().numpy(), rtol=1e-5, atol=1e-5)
            gi, gg = ops.grid_sampler3d_backward(g.float().to(dev), x.float().to(dev), grid.float().to(dev), 0, pad, align)
            np.testing.assert_allclose(gi.cpu().numpy(), xt.grad.float().numpy(), rtol=1e-5, atol=1e-5)
            np.testing.assert_allclose(gg.cpu().numpy(), gt.grad.float().numpy(), rtol=1e-4, atol=1e-4)
    # nearest forward against torch (points away from the rounding ties)
    yn = ops.grid_sampler3d(x.float().to(dev), grid.float().to(dev), 1, 0, False)
    tn = F.grid_sample(x.float(), grid.float(), mode="nearest", padding_mode="zeros", align_corners=False)
    assert torch.equal(yn.cpu(), tn)
    # NDHWC tensors are the same operator on permuted memory
    xl = x.float().permute(0, 2, 3, 4, 1).contiguous().to(dev)
    yl = ops.grid_sampler3d(xl, grid.float().to(dev), 0, 0, False, fmt="NDHWC")
    y = ops.grid_sampler3d(x.float().to(dev), grid.float().to(dev), 0, 0, False)
    assert torch.equal(yl.permute(0, 4, 1, 2, 3), y)
    # a non-finite grid value: zeros padding drops the sample (position -100), border clips it to 0
    bad = grid.float().clone()
    bad[0, 0, 0, 0, 0] = float("nan")
    bad[1, 1, 1, 1, 2] = float("inf")
    for pad in (0, 1, 2):
        y = ops.grid_sampler3d(x.float().to(dev), bad.to(dev), 0, pad, False)
        assert np.array_equal(y.cpu().numpy(), oracle.grid_sampler3d_fwd(x.float().numpy(), bad.numpy(), pad, False))
    e = ops.grid_sampler3d(torch.zeros((0, 3, 4, 4, 4), device=dev), torch.zeros((0, 2, 2, 2, 3), device=dev))
    assert e.shape == (0, 3, 2, 2, 2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("channels", [8, 6, 5])   # channel vectors of 4, 2 and 1
@pytest.mark.parametrize("interp", [0, 1])
@pytest.mark.parametrize("pad", [0, 2])
def test_grid_sampler3d_channels_last(ops, oracle, dev, dtype, channels, interp, pad):
    """NDHWC tensors run on kernels that read a tap as one contiguous run of channels: the forward keeps the oracle's
    bits, grad_grid too, grad_input is the same atomic sum as for NCDHW."""
    x, x32 = quant(torch.randn((2, channels, 5, 6, 7), generator=gen(120)), dtype)
    grid, g32 = quant(make_grid(2, 3, 4, 5, 121), dtype)
    go, go32 = quant(torch.randn((2, channels, 3, 4, 5), generator=gen(122)), dtype)
    cl = lambda t: t.permute(0, 2, 3, 4, 1).contiguous().to(dev)  # noqa: E731
    y = ops.grid_sampler3d(cl(x), grid.to(dev), interp, pad, False, fmt="NDHWC").permute(0, 4, 1, 2, 3)
    if interp == 0:
        check(y, oracle.grid_sampler3d_fwd(x32, g32, pad, False), dtype, exact=(dtype == torch.float32))
    else:
        assert torch.equal(y, ops.grid_sampler3d(x.to(dev), grid.to(dev), interp, pad, False))
    gi, gg = ops.grid_sampler3d_backward(cl(go), cl(x), grid.to(dev), interp, pad, False, fmt="NDHWC")
    ri, rg = oracle.grid_sampler3d_bwd(go32, x32, g32, interp, pad, False)
    gi = gi.permute(0, 4, 1, 2, 3)
    if dtype == torch.float32:
        np.testing.assert_allclose(gi.cpu().numpy(), ri, rtol=1e-5, atol=1e-6 * max(1.0, float(np.abs(ri).max())))
        assert np.array_equal(gg.cpu().numpy(), rg)
    else:
        check(gg, rg, dtype)
        step = np.maximum(np.abs(ri) * (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10), 1e-6 * max(1.0, float(np.abs(ri).max())))
        assert (np.abs(gi.float().cpu().numpy() - ri) <= step * 1.01 + 1e-6).all()
    # a strided channels-last view (cropped W) goes through the staging copies and gives the same result
    base = torch.zeros((2, 5, 6, 9, channels), dtype=dtype)
    base[:, :, :, 1:8, :] = x.permute(0, 2, 3, 4, 1)
    yv = ops.grid_sampler3d(base.to(dev)[:, :, :, 1:8, :], grid.to(dev), interp, pad, False, fmt="NDHWC")
    assert torch.equal(yv.permute(0, 4, 1, 2, 3), y)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("channels", [16, 20, 40])
@pytest.mark.parametrize("interp", [0, 1])
def test_grid_sampler3d_ncdhw_through_channels_last(ops, oracle, dev, dtype, channels, interp):
    """NCDHW tensors with sixteen or more channels (a multiple of four) are turned channels-last in the workspace,
    sampled by the channels-last kernels and turned back: the same bits as the oracle in the forward and for
    grad_grid, the same atomic sum for grad_input."""
    x, x32 = quant(torch.randn((2, channels, 5, 6, 7), generator=gen(130)), dtype)
    grid, g32 = quant(make_grid(2, 3, 4, 5, 131), dtype)
    go, go32 = quant(torch.randn((2, channels, 3, 4, 5), generator=gen(132)), dtype)
    for pad in (0, 1, 2):
        y = ops.grid_sampler3d(x.to(dev), grid.to(dev), interp, pad, True)
        if interp == 0:
            check(y, oracle.grid_sampler3d_fwd(x32, g32, pad, True), dtype, exact=(dtype == torch.float32))
        gi, gg = ops.grid_sampler3d_backward(go.to(dev), x.to(dev), grid.to(dev), interp, pad, True)
        ri, rg = oracle.grid_sampler3d_bwd(go32, x32, g32, interp, pad, True)
        if dtype == torch.float32:
            np.testing.assert_allclose(gi.cpu().numpy(), ri, rtol=1e-5, atol=1e-6 * max(1.0, float(np.abs(ri).max())))
            assert np.array_equal(gg.cpu().numpy(), rg)
        else:
            check(gg, rg, dtype)
            step = np.maximum(np.abs(ri) * (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10), 1e-6 * max(1.0, float(np.abs(ri).max())))
            assert (np.abs(gi.float().cpu().numpy() - ri) <= step * 1.01 + 1e-6).all()
    # masks still hold
    keep = torch.full_like(x, 7.0).to(dev)
    ops.grid_sampler3d_backward(go.to(dev), x.to(dev), grid.to(dev), interp, 0, False, mask=(False, True), input_grad=keep)
    assert torch.equal(keep.cpu(), torch.full_like(x, 7.0))
