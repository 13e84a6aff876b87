"""aclnnResize through the C ABI: "nearest" gives UpsampleNearest2d's bits and "bilinear" UpsampleBilinear2d's
(align_corners = false), both checked against the oracle."""
import numpy as np
import pytest
import torch

from test_gpu_parity import DTYPES, check, gen, nhwc, quant

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("fmt", ["NCHW", "NHWC"])
@pytest.mark.parametrize("case", [((2, 3, 8, 10), (2.0, 2.0)), ((1, 4, 7, 9), (2.15, 2.25)), ((1, 2, 16, 24), (0.32, 0.3)),
                                  ((1, 2, 5, 6), (1.0, 1.0))])
def test_resize_modes(ops, oracle, dev, dtype, fmt, case):
    shape, (sh, sw) = case
    n, c, hi, wi = shape
    ho, wo = int(hi * sh), int(wi * sw)
    x, x32 = quant(torch.randn(shape, generator=gen(80)), dtype)
    xl = torch.from_numpy(nhwc(x32) if fmt == "NHWC" else x32).to(dtype).to(dev)
    scales = (1.0, sh, sw, 1.0) if fmt == "NHWC" else (1.0, 1.0, sh, sw)
    ofmt = oracle.NHWC if fmt == "NHWC" else oracle.NCHW
    xin = nhwc(x32) if fmt == "NHWC" else x32
    y = ops.resize(xl, scales, "nearest", fmt)
    check(y, oracle.nearest2d_fwd(xin, (ho, wo), fmt=ofmt), dtype, exact=True)
    assert torch.equal(y, ops.upsample_nearest2d(xl, (ho, wo), fmt))
    y = ops.resize(xl, scales, "bilinear", fmt)
    check(y, oracle.bilinear2d_fwd(xin, (ho, wo), False, fmt=ofmt), dtype, exact=(dtype == torch.float32))
    assert torch.equal(y, ops.upsample_bilinear2d(xl, (ho, wo), False, fmt))
