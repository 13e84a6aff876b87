"""Seeded random shapes, layouts and alignments of the 3-D resamplers against the oracle: whole-number factors (the
replicate / pool kernels), ragged scales, one-axis and copy cases of the trilinear operator, channels-last packs of
every width, tensors carved out of larger buffers at odd element offsets, and strided 5-D views."""
import numpy as np
import pytest
import torch

from test_gpu_parity import check, quant
from test_gpu_random_shapes import carve

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def pick_sizes(rng):
    kind = rng.integers(0, 6)
    if kind == 0:
        a = int(rng.integers(1, 12))
        return a, a * int(rng.integers(1, 4))
    if kind == 1:
        a = int(rng.integers(1, 10))
        return a * int(rng.integers(2, 4)), a
    if kind == 2:
        a = int(rng.integers(1, 16))
        return a, a
    if kind == 3:
        return int(rng.integers(1, 3)), int(rng.integers(1, 20))
    return int(rng.integers(1, 20)), int(rng.integers(1, 20))


def cl(a):
    return np.ascontiguousarray(np.transpose(a, (0, 2, 3, 4, 1)))


@pytest.mark.parametrize("seed", range(36))
def test_upsample3d_random(ops, oracle, dev, seed):
    rng = np.random.default_rng(3000 + seed)
    dtype = DTYPES[seed % 3]
    fmt = "NDHWC" if rng.integers(0, 3) == 0 else "NCDHW"
    n, c = int(rng.integers(1, 3)), int(rng.integers(1, 10))
    (di, do), (hi, ho), (wi, wo) = pick_sizes(rng), pick_sizes(rng), pick_sizes(rng)
    if seed % 4 == 0:
        wo = 2 * wi   # the replicate / pool kernels
    align = bool(rng.integers(0, 2))
    exact = bool(rng.integers(0, 2))
    g = torch.Generator().manual_seed(seed)
    ofmt = oracle.NHWC if fmt == "NDHWC" else oracle.NCHW
    x, x32 = quant(torch.randn((n, c, di, hi, wi), generator=g), dtype)
    go, go32 = quant(torch.randn((n, c, do, ho, wo), generator=g), dtype)
    xin = cl(x32) if fmt == "NDHWC" else x32
    gin = cl(go32) if fmt == "NDHWC" else go32
    xd = carve(torch.from_numpy(xin).to(dtype), dev, rng)
    gd = carve(torch.from_numpy(gin).to(dtype), dev, rng)
    size = (do, ho, wo)
    in_shape = (n, di, hi, wi, c) if fmt == "NDHWC" else (n, c, di, hi, wi)
    # nearest / nearest-exact: copies and window sums in a fixed order
    y = ops.upsample_nearest3d(xd, size, fmt, exact=exact)
    check(y, oracle.nearest3d_fwd(xin, size, exact=exact, fmt=ofmt), dtype, exact=True)
    gi = ops.upsample_nearest3d_backward(gd, size, in_shape, fmt, exact=exact)
    check(gi, oracle.nearest3d_bwd(gin, (di, hi, wi), exact=exact, fmt=ofmt), dtype, exact=True)
    # trilinear
    y = ops.upsample_trilinear3d(xd, size, align, fmt)
    loop = oracle.trilinear3d_fwd_loop((di, hi, wi), size, align)
    check(y, oracle.trilinear3d_fwd(xin, size, align, fmt=ofmt), dtype, exact=(dtype == torch.float32 or loop == "copy"))
    gi = ops.upsample_trilinear3d_backward(gd, size, (n, c, di, hi, wi), align, fmt)
    check(gi, oracle.trilinear3d_bwd(gin, (di, hi, wi), align, fmt=ofmt), dtype, exact=(dtype == torch.float32))


@pytest.mark.parametrize("seed", range(12))
def test_views5d_random(ops, oracle, dev, seed):
    """Strided 5-D views (crops and steps on H and W, channel slices) go through the staging copies of the 3-D
    operators: the result of the call on a contiguous copy, and nothing outside a strided output view is touched."""
    rng = np.random.default_rng(4000 + seed)
    dtype = DTYPES[seed % 3]
    n, c, d = int(rng.integers(1, 3)), int(rng.integers(2, 7)), int(rng.integers(1, 6))
    h, w = int(rng.integers(4, 14)), int(rng.integers(4, 14))
    base = torch.randn((n, c, d, h + 3, 2 * w + 2), generator=torch.Generator().manual_seed(seed)).to(dtype).to(dev)
    step = int(rng.integers(1, 3))
    view = base[:, :, :, 1:1 + h, 1:1 + step * w:step]
    assert not view.is_contiguous()
    size = (int(rng.integers(1, 8)), int(rng.integers(1, 20)), int(rng.integers(1, 20)))
    dense = view.contiguous()
    assert torch.equal(ops.upsample_nearest3d(view, size), ops.upsample_nearest3d(dense, size))
    assert torch.equal(ops.upsample_trilinear3d(view, size, False), ops.upsample_trilinear3d(dense, size, False))
    out_base = torch.full((n, c, size[0], size[1], 2 * size[2]), 3.0, dtype=dtype, device=dev)
    out = out_base[..., ::2]
    ops.upsample_trilinear3d(view, size, True, out=out)
    assert torch.equal(out, ops.upsample_trilinear3d(dense, size, True))
    assert float((out_base[..., 1::2] - 3.0).abs().max()) == 0.0
    g = torch.randn((n, c) + size, generator=torch.Generator().manual_seed(seed + 1)).to(dtype).to(dev)
    gi_base = torch.zeros_like(base)
    gi = gi_base[:, :, :, 1:1 + h, 1:1 + step * w:step]
    ops.upsample_trilinear3d_backward(g, size, tuple(view.shape), False, out=gi)
    assert torch.equal(gi, ops.upsample_trilinear3d_backward(g, size, tuple(view.shape), False))
