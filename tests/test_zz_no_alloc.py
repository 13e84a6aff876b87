"""opscvUpsampleBilinear2dNoAlloc through the C ABI: the allocation-free bilinear forward must agree with the
two-phase entry point it shadows. Collected last (file name), so it runs after every other GPU test has used the
device, and it also passes when run alone."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

CASES = [
    # dtype, fmt, shape (n, c, h, w), out_hw, align, scales
    (torch.float32, "NCHW", (2, 3, 17, 23), (40, 31), False, (0.0, 0.0)),
    (torch.float32, "NCHW", (1, 4, 32, 32), (64, 64), True, (0.0, 0.0)),
    (torch.float16, "NCHW", (2, 5, 20, 24), (13, 11), False, (0.65, 0.0)),
    (torch.bfloat16, "NHWC", (2, 16, 9, 12), (18, 24), False, (2.0, 2.0)),
    (torch.float32, "NHWC", (1, 7, 11, 5), (6, 13), True, (0.0, 0.0)),
]


@pytest.mark.parametrize("dtype,fmt,shape,out_hw,align,scales", CASES)
def test_no_alloc_matches_two_phase(ops, dev, dtype, fmt, shape, out_hw, align, scales):
    gen = torch.Generator().manual_seed(90)
    n, c, h, w = shape
    x = torch.randn((n, h, w, c) if fmt == "NHWC" else shape, generator=gen).to(dtype).to(dev)
    want = ops.upsample_bilinear2d(x, out_hw, align, fmt, scales)
    # two calls in a row on the same stream: the second reuses (and rewrites) the shared tap tables
    for _ in range(2):
        got = ops.upsample_bilinear2d_no_alloc(x, out_hw, align, fmt, scales)
        torch.cuda.synchronize(dev)
        if dtype == torch.float32:
            np.testing.assert_allclose(got.cpu().numpy(), want.cpu().numpy(), rtol=1e-5, atol=1e-6)
        else:
            diff = (got.float() - want.float()).abs().max().item()
            eps = 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7
            assert diff <= eps * max(1.0, want.float().abs().max().item())


def test_no_alloc_changing_shapes_back_to_back(ops, dev):
    """Different extents in consecutive calls on one stream: each call must see its own tables."""
    gen = torch.Generator().manual_seed(91)
    a = torch.randn((1, 2, 8, 8), generator=gen).to(dev)
    b = torch.randn((1, 2, 30, 14), generator=gen).to(dev)
    ga = ops.upsample_bilinear2d_no_alloc(a, (16, 16))
    gb = ops.upsample_bilinear2d_no_alloc(b, (7, 33))
    ga2 = ops.upsample_bilinear2d_no_alloc(a, (16, 16))
    torch.cuda.synchronize(dev)
    np.testing.assert_allclose(ga.cpu().numpy(), ops.upsample_bilinear2d(a, (16, 16)).cpu().numpy(), rtol=1e-5,
                               atol=1e-6)
    np.testing.assert_allclose(gb.cpu().numpy(), ops.upsample_bilinear2d(b, (7, 33)).cpu().numpy(), rtol=1e-5,
                               atol=1e-6)
    assert torch.equal(ga, ga2)


def test_no_alloc_rejects_oversize_and_null(ops, dev):
    x = torch.zeros((1, 1, 4, 4), device=dev)
    with pytest.raises(ops.AclnnError) as err:
        ops.upsample_bilinear2d_no_alloc(x, (8193, 4), out=torch.zeros((1, 1, 1, 1), device=dev))
    assert err.value.status == 161002 and "8192" in str(err.value)
    status = ops.lib().opscvUpsampleBilinear2dNoAlloc(None, None, 0, 0, 1, 1, 4, 4, 8, 8, False, 0.0, 0.0, None)
    assert status == 161001
