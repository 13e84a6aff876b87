"""Seeded random shapes, scales, layouts and alignments against the oracle.

The fixed cases of test_gpu_parity.py pin the documented behaviours; this file sweeps the schedule choosers (integer
factors, 2x patterns, staged and direct kernels, vector widths, 16- and 32-byte store paths) with shapes nobody
picked by hand. Tensors are carved out of larger buffers at odd element offsets, so base pointers are often not
16-byte aligned and rows start at arbitrary alignments.
"""
import numpy as np
import pytest
import torch

from test_gpu_parity import check, check_sum, quant

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def carve(t, dev, rng):
    """A contiguous device copy of t that starts `off` elements into a larger buffer (off in 0..9)."""
    off = int(rng.integers(0, 10))
    buf = torch.empty(t.numel() + 16, dtype=t.dtype, device=dev)
    view = buf[off:off + t.numel()].view(t.shape)
    view.copy_(t)
    return view


def pick_sizes(rng):
    """(in, out) extents: integer factors, near-integer, arbitrary up and down scales, tiny edges."""
    kind = rng.integers(0, 6)
    if kind == 0:
        a = int(rng.integers(1, 24))
        return a, a * int(rng.integers(1, 5))
    if kind == 1:
        a = int(rng.integers(2, 24))
        return a * int(rng.integers(2, 4)), a
    if kind == 2:
        return int(rng.integers(1, 4)), int(rng.integers(1, 40))
    if kind == 3:
        return int(rng.integers(8, 72)), int(rng.integers(1, 4))
    return int(rng.integers(1, 72)), int(rng.integers(1, 72))


@pytest.mark.parametrize("seed", range(40))
def test_upsample_random(ops, oracle, dev, seed):
    rng = np.random.default_rng(1000 + seed)
    dtype = DTYPES[seed % 3]
    fmt = "NHWC" if rng.integers(0, 3) == 0 else "NCHW"
    n, c = int(rng.integers(1, 4)), int(rng.integers(1, 20))
    (hi, ho), (wi, wo) = pick_sizes(rng), pick_sizes(rng)
    align = bool(rng.integers(0, 2))
    g = torch.Generator().manual_seed(seed)
    shape_in = (n, hi, wi, c) if fmt == "NHWC" else (n, c, hi, wi)
    shape_out = (n, ho, wo, c) if fmt == "NHWC" else (n, c, ho, wo)
    ofmt = oracle.NHWC if fmt == "NHWC" else oracle.NCHW
    x, x32 = quant(torch.randn(shape_in, generator=g), dtype)
    go, go32 = quant(torch.randn(shape_out, generator=g), dtype)
    xd, god = carve(x, dev, rng), carve(go, dev, rng)
    in_size = (n, hi, wi, c) if fmt == "NHWC" else (n, c, hi, wi)
    # nearest
    y = ops.upsample_nearest2d(xd, (ho, wo), fmt)
    check(y, oracle.nearest2d_fwd(x32, (ho, wo), fmt=ofmt), dtype, exact=True)
    gi = ops.upsample_nearest2d_backward(god, (ho, wo), in_size, fmt)
    check(gi, oracle.nearest2d_bwd(go32, (hi, wi), fmt=ofmt), dtype, exact=True)  # the reference's summation order
    # bilinear
    y = ops.upsample_bilinear2d(xd, (ho, wo), align, fmt)
    check(y, oracle.bilinear2d_fwd(x32, (ho, wo), align, fmt=ofmt), dtype, exact=(dtype == torch.float32))
    gi = ops.upsample_bilinear2d_backward(god, (ho, wo), in_size, align, fmt)
    check_sum(gi, oracle.bilinear2d_bwd(go32, (hi, wi), align, fmt=ofmt), dtype)
    if fmt == "NCHW":
        y = ops.upsample_bicubic2d_aa(xd, (ho, wo), align)
        check_sum(y, oracle.bicubic_aa_fwd(x32, (ho, wo), align), dtype)
        gi = ops.upsample_bicubic2d_aa_grad(god, (ho, wo), in_size, align)
        check_sum(gi, oracle.bicubic_aa_bwd(go32, (hi, wi), align), dtype)


@pytest.mark.parametrize("seed", range(12))
def test_upsample_streaming_shapes(ops, oracle, dev, seed):
    """Down-scales with rows that are multiples of 8: the streaming bicubic-AA kernels; and 2x up-scales with rows that
    are multiples of 4 or 8: the input-major bilinear and nearest kernels, with and without 32-byte aligned rows."""
    rng = np.random.default_rng(2000 + seed)
    dtype = DTYPES[seed % 3]
    n, c = int(rng.integers(1, 3)), int(rng.integers(1, 40))
    wi = 8 * int(rng.integers(1, 40))
    hi = int(rng.integers(20, 90))
    ho, wo = max(1, int(hi / rng.uniform(1.0, 5.0))), max(1, int(wi / rng.uniform(1.0, 5.0)))
    g = torch.Generator().manual_seed(seed)
    x, x32 = quant(torch.rand((n, c, hi, wi), generator=g), dtype)
    go, go32 = quant(torch.randn((n, c, ho, wo), generator=g), dtype)
    y = ops.upsample_bicubic2d_aa(carve(x, dev, rng), (ho, wo), False)
    check_sum(y, oracle.bicubic_aa_fwd(x32, (ho, wo), False), dtype)
    gi = ops.upsample_bicubic2d_aa_grad(carve(go, dev, rng), (ho, wo), (n, c, hi, wi), False)
    check_sum(gi, oracle.bicubic_aa_bwd(go32, (hi, wi), False), dtype)
    # 2x
    w2 = 4 * int(rng.integers(1, 30))
    h2 = int(rng.integers(2, 40))
    x, x32 = quant(torch.randn((n, c, h2, w2), generator=g), dtype)
    go, go32 = quant(torch.randn((n, c, 2 * h2, 2 * w2), generator=g), dtype)
    xd, god = carve(x, dev, rng), carve(go, dev, rng)
    y = ops.upsample_nearest2d(xd, (2 * h2, 2 * w2), scales=(2.0, 2.0))
    check(y, oracle.nearest2d_fwd(x32, (2 * h2, 2 * w2), (2.0, 2.0)), dtype, exact=True)
    y = ops.upsample_bilinear2d(xd, (2 * h2, 2 * w2), False)
    check(y, oracle.bilinear2d_fwd(x32, (2 * h2, 2 * w2), False), dtype, exact=(dtype == torch.float32))
    gi = ops.upsample_bilinear2d_backward(god, (2 * h2, 2 * w2), (n, c, h2, w2), False)
    check_sum(gi, oracle.bilinear2d_bwd(go32, (h2, w2), False), dtype)
    gi = ops.upsample_nearest2d_backward(god, (2 * h2, 2 * w2), (n, c, h2, w2), scales=(2.0, 2.0))
    check(gi, oracle.nearest2d_bwd(go32, (h2, w2), (2.0, 2.0)), dtype, exact=True)


@pytest.mark.parametrize("seed", range(24))
def test_grid_sampler_random(ops, oracle, dev, seed):
    rng = np.random.default_rng(3000 + seed)
    dtype = DTYPES[seed % 3]
    big = seed % 2 == 0  # enough (image, channel group) blocks for the staged backward kernels
    n = int(rng.integers(4, 9)) if big else int(rng.integers(1, 4))
    c = int(rng.integers(70, 100)) if big else int(rng.integers(1, 12))
    hi, wi = int(rng.integers(1, 20)), int(rng.integers(1, 20))
    ho, wo = int(rng.integers(1, 24)), int(rng.integers(1, 24))
    interp = 0 if big else int(rng.integers(0, 2))
    pad, align = int(rng.integers(0, 3)), bool(rng.integers(0, 2))
    g = torch.Generator().manual_seed(seed)
    x, x32 = quant(torch.randn((n, c, hi, wi), generator=g), dtype)
    grid, grid32 = quant(torch.rand((n, ho, wo, 2), generator=g) * 2.6 - 1.3, dtype)
    go, go32 = quant(torch.randn((n, c, ho, wo), generator=g), dtype)
    xd, gd, god = carve(x, dev, rng), carve(grid, dev, rng), carve(go, dev, rng)
    y = ops.grid_sampler2d(xd, gd, interp, pad, align)
    check(y, oracle.grid_sampler2d_fwd(x32, grid32, interp, pad, align), dtype, exact=(dtype == torch.float32))
    ri, rg = oracle.grid_sampler2d_bwd(go32, x32, grid32, interp, pad, align)
    for det in (False, True):
        ops.set_deterministic(det)
        try:
            gi, gg = ops.grid_sampler2d_backward(god, xd, gd, interp, pad, align)
        finally:
            ops.set_deterministic(False)
        check_sum(gi, ri, dtype)
        check_sum(gg, rg, dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("fmt", ["NCHW", "NHWC"])
def test_bilinear_2x_16bit_forward_is_bit_exact(ops, oracle, dev, dtype, fmt):
    """Exact 2x: the weights are 0, 0.25, 0.75 and 1, so every weight * value product is exact in fp32 and the kernels
    use a fused multiply-add in the horizontal pass. That must give the oracle's bits, not only its value to 1 ulp.
    Values span many binades so that sums do round."""
    n, c, hi, wi = 3, 16, 21, 40
    g = torch.Generator().manual_seed(77)
    x = torch.randn((n, c, hi, wi), generator=g) * torch.exp2(torch.randint(-12, 12, (n, c, hi, wi), generator=g).float())
    if fmt == "NHWC":
        x = x.permute(0, 2, 3, 1).contiguous()
    xs, x32 = quant(x, dtype)
    ofmt = oracle.NHWC if fmt == "NHWC" else oracle.NCHW
    y = ops.upsample_bilinear2d(xs.to(dev), (2 * hi, 2 * wi), False, fmt)
    check(y, oracle.bilinear2d_fwd(x32, (2 * hi, 2 * wi), False, fmt=ofmt), dtype, exact=True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_bilinear_2x_tall_planes(ops, oracle, dev, dtype):
    """Planes taller than one tile of the 2x kernels (forward: 512 output rows per tile; backward: as many rows as fit
    the shared-memory budget), few planes, so every block's run crosses tile and plane-group borders."""
    n, c, hi, wi = 1, 3, 700, 16
    g = torch.Generator().manual_seed(78)
    x, x32 = quant(torch.randn((n, c, hi, wi), generator=g), dtype)
    go, go32 = quant(torch.randn((n, c, 2 * hi, 2 * wi), generator=g), dtype)
    y = ops.upsample_bilinear2d(x.to(dev), (2 * hi, 2 * wi), False)
    check(y, oracle.bilinear2d_fwd(x32, (2 * hi, 2 * wi), False), dtype, exact=(dtype == torch.float32))
    gi = ops.upsample_bilinear2d_backward(go.to(dev), (2 * hi, 2 * wi), (n, c, hi, wi), False)
    check_sum(gi, oracle.bilinear2d_bwd(go32, (hi, wi), False), dtype)
