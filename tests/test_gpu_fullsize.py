"""GPU parity at the full sizes of the benchmark configurations.

The oracle is a scalar CPU program, so at these sizes it checks the first and the last image of the batch only
(every operator is independent per image, so those two slices exercise the largest offsets), and size-independent
properties cover the rest of the tensor:
  * nearest 2x: backward(forward(x)) == 4 * x exactly (four equal copies summed);
  * interpolation weights of an output sum to one, so a constant image maps to the same constant, and the sum
    of a gradient is preserved by every backward;
  * the reproducible modes give identical bits twice; the atomic and the reproducible grid-sampler backward agree.
"""
import numpy as np
import pytest
import torch

from test_gpu_parity import check, check_sum, gen

pytestmark = pytest.mark.gpu


def ends(t):
    """First and last image of a batch-major tensor, as one CPU tensor."""
    return torch.cat([t[:1], t[-1:]]).cpu()


def test_cfg2_fpn_upsample_fp16(ops, oracle, dev):
    n, c, hi, wi, ho, wo = 32, 256, 56, 56, 112, 112
    x = torch.randn((n, c, hi, wi), generator=gen(1236)).to(torch.float16)
    go = torch.randn((n, c, ho, wo), generator=gen(1237)).to(torch.float16)
    xd, god = x.to(dev), go.to(dev)
    # nearest
    yn = ops.upsample_nearest2d(xd, (ho, wo), scales=(2.0, 2.0))
    check(ends(yn), oracle.nearest2d_fwd(ends(x).float().numpy(), (ho, wo), (2.0, 2.0)), torch.float16, exact=True)
    back = ops.upsample_nearest2d_backward(yn, (ho, wo), (n, c, hi, wi), scales=(2.0, 2.0))
    assert torch.equal(back.cpu(), (x.float() * 4).to(torch.float16))
    gn = ops.upsample_nearest2d_backward(god, (ho, wo), (n, c, hi, wi), scales=(2.0, 2.0))
    # the kernel adds the four fp32 values in the reference's row-major order: same bits
    check(ends(gn), oracle.nearest2d_bwd(ends(go).float().numpy(), (hi, wi), (2.0, 2.0)), torch.float16, exact=True)
    # bilinear
    yb = ops.upsample_bilinear2d(xd, (ho, wo), False, scales=(2.0, 2.0))
    check(ends(yb), oracle.bilinear2d_fwd(ends(x).float().numpy(), (ho, wo), False, (2.0, 2.0)), torch.float16)
    const = torch.full((n, c, hi, wi), 0.75, dtype=torch.float16, device=dev)
    assert torch.equal(ops.upsample_bilinear2d(const, (ho, wo), False, scales=(2.0, 2.0)),
                       torch.full((n, c, ho, wo), 0.75, dtype=torch.float16, device=dev))
    gb = ops.upsample_bilinear2d_backward(god, (ho, wo), (n, c, hi, wi), False, scales=(2.0, 2.0))
    gb2 = ops.upsample_bilinear2d_backward(god, (ho, wo), (n, c, hi, wi), False, scales=(2.0, 2.0))
    assert torch.equal(gb.view(torch.int16), gb2.view(torch.int16))
    # the reference runs its gather ("determine") kernel for this call (up-scale, user scale equal to the size
    # ratio): at most 1 ulp of fp16 from it, and from the atomic kernel's serial order as well
    go_ends = ends(go).float().numpy()
    assert oracle.bilinear2d_bwd_kernel_choice((hi, wi), (ho, wo), False, (2.0, 2.0)) == "gather"
    check(ends(gb), oracle.bilinear2d_bwd(go_ends, (hi, wi), False, (2.0, 2.0), definition="gather"), torch.float16)
    check(ends(gb), oracle.bilinear2d_bwd(go_ends, (hi, wi), False, (2.0, 2.0), definition="scatter"), torch.float16)
    # per-plane sums are preserved (fp32 sums of the fp16 tensors; the fp16 rounding of gi bounds the difference)
    s_in, s_out = god.float().sum((2, 3)), gb.float().sum((2, 3))
    assert (s_in - s_out).abs().max().item() <= 2.0 ** -10 * gb.float().abs().sum((2, 3)).max().item()


def test_adj2_bicubic_2x_fp16(ops, oracle, dev):
    """The exactly-2x bicubic kernels at the benchmark shapes: first and last image against the oracle, a constant
    image stays constant (the four coefficients of a set sum to one up to their rounding), the backward preserves
    the sum of the gradient per plane, and a second call gives the same bits."""
    n, c, hi, wi, ho, wo = 32, 256, 56, 56, 112, 112
    x = torch.randn((n, c, hi, wi), generator=gen(1260)).to(torch.float16)
    go = torch.randn((n, c, ho, wo), generator=gen(1261)).to(torch.float16)
    xd, god = x.to(dev), go.to(dev)
    y = ops.upsample_bicubic2d(xd, (ho, wo), False)
    check(ends(y), oracle.bicubic2d_fwd(ends(x).float().numpy(), (ho, wo), False), torch.float16)
    const = ops.upsample_bicubic2d(torch.full((n, c, hi, wi), 0.75, dtype=torch.float16, device=dev), (ho, wo), False)
    assert (const.float() - 0.75).abs().max().item() <= 2.0 ** -11
    gi = ops.upsample_bicubic2d_backward(god, (ho, wo), (n, c, hi, wi), False)
    assert torch.equal(gi.view(torch.int16),
                       ops.upsample_bicubic2d_backward(god, (ho, wo), (n, c, hi, wi), False).view(torch.int16))
    check(ends(gi), oracle.bicubic2d_bwd(ends(go).float().numpy(), (hi, wi), False, definition="gather"), torch.float16)
    s_in, s_out = god.float().sum((2, 3)), gi.float().sum((2, 3))
    assert (s_in - s_out).abs().max().item() <= 2.0 ** -9 * gi.float().abs().sum((2, 3)).max().item()


def test_cfg3_bicubic_aa_fp32(ops, oracle, dev):
    n, c, hi, wi, ho, wo = 64, 3, 1024, 1024, 224, 224
    x = torch.randint(0, 256, (n, c, hi, wi), generator=gen(1238)).float() / 255
    go = torch.randn((n, c, ho, wo), generator=gen(1239))
    xd, god = x.to(dev), go.to(dev)
    y = ops.upsample_bicubic2d_aa(xd, (ho, wo), False)
    check(ends(y), oracle.bicubic_aa_fwd(ends(x).numpy(), (ho, wo), False), torch.float32)
    const = ops.upsample_bicubic2d_aa(torch.full((2, 1, hi, wi), 0.625, device=dev), (ho, wo), False)
    assert (const - 0.625).abs().max().item() <= 1e-6
    gi = ops.upsample_bicubic2d_aa_grad(god, (ho, wo), (n, c, hi, wi), False)
    check(ends(gi), oracle.bicubic_aa_bwd(ends(go).numpy(), (hi, wi), False), torch.float32)
    s_in, s_out = god.double().sum((2, 3)), gi.double().sum((2, 3))
    assert (s_in - s_out).abs().max().item() <= 1e-4 * god.double().abs().sum((2, 3)).max().item()
    assert ops.async_copy_timeouts() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cfg4_grid_sampler(ops, oracle, dev, dtype):
    n, c, hi, wi, ho, wo = 16, 256, 64, 64, 128, 128
    x = torch.randn((n, c, hi, wi), generator=gen(1240)).to(dtype)
    grid = (torch.rand((n, ho, wo, 2), generator=gen(1241)) * 2.2 - 1.1).to(dtype)
    go = torch.randn((n, c, ho, wo), generator=gen(1242)).to(dtype)
    xd, gd, god = x.to(dev), grid.to(dev), go.to(dev)
    x32, g32, go32 = ends(x).float().numpy(), ends(grid).float().numpy(), ends(go).float().numpy()
    y = ops.grid_sampler2d(xd, gd, 0, 0, False)
    check(ends(y), oracle.grid_sampler2d_fwd(x32, g32, 0, 0, False), dtype, exact=(dtype == torch.float32))
    ri, rg = oracle.grid_sampler2d_bwd(go32, x32, g32, 0, 0, False)
    gi_a, gg_a = ops.grid_sampler2d_backward(god, xd, gd, 0, 0, False)
    check_sum(ends(gi_a), ri, dtype)
    check_sum(ends(gg_a), rg, dtype)
    ops.set_deterministic(True)
    try:
        gi_d, gg_d = ops.grid_sampler2d_backward(god, xd, gd, 0, 0, False)
        gi_e, gg_e = ops.grid_sampler2d_backward(god, xd, gd, 0, 0, False)
    finally:
        ops.set_deterministic(False)
    bits = torch.int32 if dtype == torch.float32 else torch.int16
    assert torch.equal(gi_d.view(bits), gi_e.view(bits)) and torch.equal(gg_d.view(bits), gg_e.view(bits))
    check_sum(ends(gi_d), ri, dtype)
    check_sum(ends(gg_d), rg, dtype)
    # the two modes agree over the whole tensor
    tol = 1e-5 if dtype == torch.float32 else 2.0 ** -7
    scale = gi_d.float().abs().max().item()
    assert (gi_a.float() - gi_d.float()).abs().max().item() <= tol * scale


def test_cfg5_box_sweep_shard(ops, oracle, dev):
    # bilinear bf16 NHWC: one eighth of the box-level batch (the per-GPU shard at 8 GPUs)
    n, c, hi, wi, ho, wo = 64, 256, 64, 64, 128, 128
    x = torch.randn((n, hi, wi, c), generator=gen(1243)).to(torch.bfloat16)
    y = ops.upsample_bilinear2d(x.to(dev), (ho, wo), False, "NHWC")
    ref = oracle.bilinear2d_fwd(ends(x).float().numpy(), (ho, wo), False, fmt=oracle.NHWC)
    check(ends(y), ref, torch.bfloat16)
    # grid sampler fp32 with affine grids
    n2, c2, h2 = 32, 128, 96
    g = gen(1244)
    phi = (torch.rand(n2, generator=g) * 60 - 30) * np.pi / 180
    s = torch.rand(n2, generator=g) * 0.4 + 0.8
    t = torch.rand((n2, 2), generator=g) * 0.2 - 0.1
    theta = torch.stack([torch.stack([s * torch.cos(phi), -s * torch.sin(phi), t[:, 0]], 1),
                         torch.stack([s * torch.sin(phi), s * torch.cos(phi), t[:, 1]], 1)], 1)
    grid = torch.nn.functional.affine_grid(theta, (n2, c2, h2, h2), align_corners=False).contiguous()
    gx = torch.randn((n2, c2, h2, h2), generator=g)
    gy = ops.grid_sampler2d(gx.to(dev), grid.to(dev), 0, 0, False)
    check(ends(gy), oracle.grid_sampler2d_fwd(ends(gx).numpy(), ends(grid).numpy(), 0, 0, False), torch.float32,
          exact=True)


def _affine_grids(n, size, g):
    phi = (torch.rand(n, generator=g) * 60 - 30) * np.pi / 180
    s = torch.rand(n, generator=g) * 0.4 + 0.8
    t = torch.rand((n, 2), generator=g) * 0.2 - 0.1
    theta = torch.stack([torch.stack([s * torch.cos(phi), -s * torch.sin(phi), t[:, 0]], 1),
                         torch.stack([s * torch.sin(phi), s * torch.cos(phi), t[:, 1]], 1)], 1)
    return torch.nn.functional.affine_grid(theta, (n, 1, size, size), align_corners=False).contiguous()


def test_cfg5_box_sweep_whole_batch_on_one_gpu(ops, oracle, dev):
    """The one-GPU point of the box sweep: the whole batch in one call. The bilinear output has 512 * 128 * 128 * 256 =
    2^31 elements, so every element offset of the last image is at or beyond 2^31 - 2^22 and the last one is 2^31 - 1:
    in-kernel offsets must be 64-bit. The first and the last image are seeded on the CPU and checked against the
    oracle; the images between them are filled on the device (the oracle, a scalar CPU program, could not check them
    in reasonable time, and every image is computed independently)."""
    n, c, hi, wi, ho, wo = 512, 256, 64, 64, 128, 128
    x = torch.empty((n, hi, wi, c), dtype=torch.bfloat16, device=dev)
    x.normal_(generator=torch.Generator(device=dev).manual_seed(1245))
    first_last = torch.randn((2, hi, wi, c), generator=gen(1246)).to(torch.bfloat16)
    x[0].copy_(first_last[0])
    x[-1].copy_(first_last[1])
    y = ops.upsample_bilinear2d(x, (ho, wo), False, "NHWC")
    assert y.numel() == 2 ** 31
    ref = oracle.bilinear2d_fwd(first_last.float().numpy(), (ho, wo), False, fmt=oracle.NHWC)
    check(ends(y), ref, torch.bfloat16)
    # an image in the middle against a separate single-image call (same kernel, small offsets)
    mid = n // 2 + 1
    assert torch.equal(y[mid].view(torch.int16),
                       ops.upsample_bilinear2d(x[mid:mid + 1].contiguous(), (ho, wo), False, "NHWC")[0].view(torch.int16))
    del y, x
    # grid sampler fp32, N = 256, affine grids
    n2, c2, h2 = 256, 128, 96
    g = gen(1247)
    grid = _affine_grids(n2, h2, g)
    gx = torch.empty((n2, c2, h2, h2), device=dev)
    gx.normal_(generator=torch.Generator(device=dev).manual_seed(1248))
    fl = torch.randn((2, c2, h2, h2), generator=g)
    gx[0].copy_(fl[0])
    gx[-1].copy_(fl[1])
    gy = ops.grid_sampler2d(gx, grid.to(dev), 0, 0, False)
    check(ends(gy), oracle.grid_sampler2d_fwd(fl.numpy(), ends(grid).numpy(), 0, 0, False), torch.float32, exact=True)
    mid = n2 // 2 + 1
    assert torch.equal(gy[mid], ops.grid_sampler2d(gx[mid:mid + 1].contiguous(), grid[mid:mid + 1].to(dev), 0, 0, False)[0])


def test_volumes_past_two_to_the_31_elements(ops, oracle, dev):
    """3-D resamplers on an output of 2^31 + 2^24 fp16 elements (4.3 GB): offsets of the last planes need 64 bits. The
    oracle checks the first and the last plane; the rest of the tensor through size-independent properties: the 2x
    nearest backward of the forward is exactly 8 x the input, and trilinear interpolation of a constant volume gives
    the constant back."""
    n, c, di, hi, wi = 1, 129, 64, 128, 256
    do, ho, wo = 2 * di, 2 * hi, 2 * wi
    assert n * c * do * ho * wo > 2 ** 31
    x = (torch.randn((n, c, di, hi, wi), generator=gen(1250)) * 0.25).to(torch.float16)
    xd = x.to(dev)
    y = ops.upsample_nearest3d(xd, (do, ho, wo))
    for ch in (0, c - 1):
        ref = oracle.nearest3d_fwd(x[:, ch:ch + 1].float().numpy(), (do, ho, wo))
        assert np.array_equal(y[:, ch:ch + 1].float().cpu().numpy(), ref)
    back = ops.upsample_nearest3d_backward(y, (do, ho, wo), (n, c, di, hi, wi))
    assert torch.equal(back.float(), xd.float() * 8.0)   # eight equal copies: exact in fp32, and x * 8 is a power-of-two scale
    del back
    t = ops.upsample_trilinear3d(xd, (do, ho, wo), False)
    for ch in (0, c - 1):
        ref = oracle.trilinear3d_fwd(x[:, ch:ch + 1].float().numpy(), (do, ho, wo), False)
        check(t[:, ch:ch + 1], ref, torch.float16)
    gi = ops.upsample_trilinear3d_backward(t, (do, ho, wo), (n, c, di, hi, wi), False)
    for ch in (0, c - 1):
        ref = oracle.trilinear3d_bwd(t[:, ch:ch + 1].float().cpu().numpy(), (di, hi, wi), False)
        check(gi[:, ch:ch + 1], ref, torch.float16)
    del t, gi, y
    const = torch.full((n, c, di, hi, wi), 0.75, dtype=torch.float16, device=dev)
    out = ops.upsample_trilinear3d(const, (do, ho, wo), True)
    assert float(out.min()) == 0.75 and float(out.max()) == 0.75
