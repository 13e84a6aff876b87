"""opscvUpsampleBilinear2dNoAlloc through the C ABI: the allocation-free bilinear forward is held to the same bar as
the two-phase entry point it shadows: the CPU oracle's bits for fp32, at most 1 ulp of the output type for fp16 /
bf16, and the same bits as the two-phase call. Collected last (file name), so it runs after every other GPU test
has used the device, and it also passes when run alone."""
import numpy as np
import pytest
import torch

from test_gpu_parity import check

pytestmark = pytest.mark.gpu

CASES = [
    # dtype, fmt, shape (n, c, h, w), out_hw, align, scales
    (torch.float32, "NCHW", (2, 3, 17, 23), (40, 31), False, (0.0, 0.0)),
    (torch.float32, "NCHW", (1, 4, 32, 32), (64, 64), True, (0.0, 0.0)),
    (torch.float16, "NCHW", (2, 5, 20, 24), (13, 11), False, (0.65, 0.0)),
    (torch.bfloat16, "NHWC", (2, 16, 9, 12), (18, 24), False, (2.0, 2.0)),
    (torch.float32, "NHWC", (1, 7, 11, 5), (6, 13), True, (0.0, 0.0)),
    (torch.float32, "NCHW", (1, 2, 9, 7), (9, 7), False, (0.0, 0.0)),    # same extents: a copy
    (torch.float32, "NCHW", (1, 2, 9, 7), (9, 7), False, (1.7, 0.4)),    # same extents, scales that disagree: still a copy
    (torch.float16, "NHWC", (1, 3, 6, 5), (6, 5), True, (0.0, 0.0)),
]


def _oracle_ref(oracle, x, fmt, out_hw, align, scales):
    x32 = x.detach().cpu().float().numpy()
    return oracle.bilinear2d_fwd(x32, out_hw, align, scales, fmt=oracle.NHWC if fmt == "NHWC" else oracle.NCHW)


@pytest.mark.parametrize("dtype,fmt,shape,out_hw,align,scales", CASES)
def test_no_alloc_matches_oracle_and_two_phase(ops, oracle, dev, dtype, fmt, shape, out_hw, align, scales):
    gen = torch.Generator().manual_seed(90)
    n, c, h, w = shape
    x = torch.randn((n, h, w, c) if fmt == "NHWC" else shape, generator=gen).to(dtype).to(dev)
    ref = _oracle_ref(oracle, x, fmt, out_hw, align, scales)
    want = ops.upsample_bilinear2d(x, out_hw, align, fmt, scales)
    bits = torch.int32 if dtype == torch.float32 else torch.int16
    # two calls in a row on the same stream: the second reuses (and rewrites) the shared tap tables
    for _ in range(2):
        got = ops.upsample_bilinear2d_no_alloc(x, out_hw, align, fmt, scales)
        torch.cuda.synchronize(dev)
        check(got, ref, dtype, exact=(dtype == torch.float32))   # fp32: the oracle's bits; 16-bit: <= 1 ulp
        assert torch.equal(got.view(bits), want.view(bits))      # and the two-phase entry point's bits


def test_no_alloc_same_size_keeps_non_finite_values(ops, oracle, dev):
    """Equal extents copy the tensor: an Inf stays an Inf (interpolating with a zero weight would make it NaN)."""
    x = torch.randn((1, 2, 5, 6), generator=torch.Generator().manual_seed(92))
    x[0, 0, 2, 3] = float("inf")
    x[0, 1, 0, 0] = -float("inf")
    for scales in ((0.0, 0.0), (1.0, 1.0), (2.0, 0.5)):
        got = ops.upsample_bilinear2d_no_alloc(x.to(dev), (5, 6), False, "NCHW", scales)
        assert torch.equal(got.cpu(), x)
        assert torch.equal(ops.upsample_bilinear2d(x.to(dev), (5, 6), False, "NCHW", scales).cpu(), x)


def test_no_alloc_largest_extent(ops, oracle, dev):
    """outH = outW = 8192, the capacity of the built-in tables, is accepted and correct; 8193 is rejected."""
    x = torch.randn((1, 1, 3, 5), generator=torch.Generator().manual_seed(93))
    got = ops.upsample_bilinear2d_no_alloc(x.to(dev), (8192, 8192))
    torch.cuda.synchronize(dev)
    ref = oracle.bilinear2d_fwd(x.numpy(), (8192, 8192), False)
    assert np.array_equal(got.cpu().numpy(), ref)
    with pytest.raises(ops.AclnnError) as err:
        ops.upsample_bilinear2d_no_alloc(x.to(dev), (8192, 8193), out=torch.zeros((1, 1, 1, 1), device=dev))
    assert err.value.status == 161002


def test_no_alloc_changing_shapes_back_to_back(ops, oracle, dev):
    """Different extents in consecutive calls on one stream: each call must see its own tables."""
    gen = torch.Generator().manual_seed(91)
    a = torch.randn((1, 2, 8, 8), generator=gen)
    b = torch.randn((1, 2, 30, 14), generator=gen)
    ga = ops.upsample_bilinear2d_no_alloc(a.to(dev), (16, 16))
    gb = ops.upsample_bilinear2d_no_alloc(b.to(dev), (7, 33))
    ga2 = ops.upsample_bilinear2d_no_alloc(a.to(dev), (16, 16))
    torch.cuda.synchronize(dev)
    assert np.array_equal(ga.cpu().numpy(), oracle.bilinear2d_fwd(a.numpy(), (16, 16), False))
    assert np.array_equal(gb.cpu().numpy(), oracle.bilinear2d_fwd(b.numpy(), (7, 33), False))
    assert torch.equal(ga, ga2)


def test_no_alloc_rejects_oversize_and_null(ops, dev):
    x = torch.zeros((1, 1, 4, 4), device=dev)
    with pytest.raises(ops.AclnnError) as err:
        ops.upsample_bilinear2d_no_alloc(x, (8193, 4), out=torch.zeros((1, 1, 1, 1), device=dev))
    assert err.value.status == 161002 and "8192" in str(err.value)
    status = ops.lib().opscvUpsampleBilinear2dNoAlloc(None, None, 0, 0, 1, 1, 4, 4, 8, 8, False, 0.0, 0.0, None)
    assert status == 161001
