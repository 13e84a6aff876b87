"""Views that are dense in the other layout's memory order (a channels-last tensor behind an NCHW handle, an NCHW
tensor behind an NHWC handle) run on that layout's kernels in place: the same bits as the contiguous call and no
staging copies (the launch count of the call equals that of a contiguous call)."""
import pytest
import torch

from test_gpu_parity import gen

pytestmark = pytest.mark.gpu


def _launches(ops, fn):
    ops.reset_launch_count()
    out = fn()
    torch.cuda.synchronize()
    return out, ops.launch_count()


def _cases(ops):
    return [
        ("nearest", lambda x, o, f, out: ops.upsample_nearest2d(x, o, f, out=out),
         lambda g, o, s, f, out: ops.upsample_nearest2d_backward(g, o, s, f, out=out)),
        ("bilinear", lambda x, o, f, out: ops.upsample_bilinear2d(x, o, False, f, out=out),
         lambda g, o, s, f, out: ops.upsample_bilinear2d_backward(g, o, s, False, f, out=out)),
        ("bicubic", lambda x, o, f, out: ops.upsample_bicubic2d(x, o, False, f, out=out),
         lambda g, o, s, f, out: ops.upsample_bicubic2d_backward(g, o, s, False, f, out=out)),
        ("nearest_exact", lambda x, o, f, out: ops.upsample_nearest_exact2d(x, o, f, out=out), None),
    ]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 8, 9, 12, 20, 31), (1, 16, 14, 14, 28, 28), (2, 3, 16, 10, 5, 7)])
def test_channels_last_behind_an_nchw_handle(ops, dev, dtype, shape):
    n, c, hi, wi, ho, wo = shape
    x = torch.randn((n, c, hi, wi), generator=gen(90)).to(dtype).to(dev)
    g = torch.randn((n, c, ho, wo), generator=gen(91)).to(dtype).to(dev)
    for name, fwd, bwd in _cases(ops):
        want, base = _launches(ops, lambda: fwd(x, (ho, wo), "NCHW", None))
        x_cl = x.contiguous(memory_format=torch.channels_last)
        out_cl = torch.empty_like(want, memory_format=torch.channels_last)
        assert not x_cl.is_contiguous() or c == 1
        _, count = _launches(ops, lambda: fwd(x_cl, (ho, wo), "NCHW", out_cl))
        assert torch.equal(out_cl, want), name
        # the NHWC kernel on the same memory, no gather / scatter copies around it
        _, nhwc_count = _launches(ops, lambda: fwd(x.permute(0, 2, 3, 1).contiguous(), (ho, wo), "NHWC", None))
        assert count == nhwc_count, (name, count, nhwc_count, base)
        if bwd is None:
            continue
        want = bwd(g, (ho, wo), (n, c, hi, wi), "NCHW", None)
        g_cl = g.contiguous(memory_format=torch.channels_last)
        gi_cl = torch.empty_like(want, memory_format=torch.channels_last)
        _, count = _launches(ops, lambda: bwd(g_cl, (ho, wo), (n, c, hi, wi), "NCHW", gi_cl))
        _, nhwc_count = _launches(ops, lambda: bwd(g.permute(0, 2, 3, 1).contiguous(), (ho, wo), (n, hi, wi, c), "NHWC", None))
        assert count == nhwc_count, (name, count, nhwc_count)
        if name == "bilinear":   # the NHWC backward sums in another order than the NCHW one
            torch.testing.assert_close(gi_cl.float(), want.float(), rtol=1e-5 if dtype == torch.float32 else 1e-2,
                                       atol=1e-6 if dtype == torch.float32 else 2e-2)
        else:
            assert torch.equal(gi_cl, want), name


def test_nchw_memory_behind_an_nhwc_handle(ops, dev):
    x = torch.randn((2, 6, 9, 12), generator=gen(92)).to(dev)         # NCHW memory
    view = x.permute(0, 2, 3, 1)                                        # dims N, H, W, C with NCHW strides
    want = ops.upsample_bilinear2d(x, (20, 31), False, "NCHW")
    out = torch.empty((2, 6, 20, 31), device=dev).permute(0, 2, 3, 1)   # the same kind of view for the output
    _, count = _launches(ops, lambda: ops.upsample_bilinear2d(view, (20, 31), False, "NHWC", out=out))
    _, base = _launches(ops, lambda: ops.upsample_bilinear2d(x, (20, 31), False, "NCHW"))
    assert torch.equal(out.permute(0, 3, 1, 2), want) and count == base
    # same extents: a flat copy of the permuted memory
    same = torch.empty((2, 6, 9, 12), device=dev).permute(0, 2, 3, 1)
    _, count = _launches(ops, lambda: ops.upsample_bilinear2d(view, (9, 12), False, "NHWC", out=same))
    assert torch.equal(same, view) and count == 1


def test_mixed_layouts_still_go_through_staging(ops, dev):
    x = torch.randn((2, 8, 9, 12), generator=gen(93)).to(dev)
    want = ops.upsample_bilinear2d(x, (20, 31), False, "NCHW")
    x_cl = x.contiguous(memory_format=torch.channels_last)
    got = ops.upsample_bilinear2d(x_cl, (20, 31), False, "NCHW")          # contiguous NCHW output
    assert torch.equal(got, want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("align", [False, True])
def test_strided_nchw_views(ops, dev, dtype, align):
    """Crops, steps, channel slices and broadcast batches on either side of the forwards give the bits of the call on
    contiguous copies. A 2x nearest up-sample between views with unit W strides runs on the replicate kernel with
    pitches (one launch: no gather copy, no table builder, no scatter copy); everything else goes through the
    staging copies."""
    base = torch.randn((3, 6, 20, 32), generator=gen(92)).to(dtype).to(dev)
    views = {
        "crop": base[:, 1:4, 2:17, 8:24],
        "step": base[::2, :, ::2, 1::3],
        "broadcast": base[:1, :, 4:12, 8:24].expand(4, 6, 8, 16),
        "channel slice": base[:, ::2],
    }
    for name, v in views.items():
        assert not v.is_contiguous()
        dense = v.contiguous()
        for ho, wo in ((v.shape[2] * 2, v.shape[3] * 2), (v.shape[2] * 3, v.shape[3] * 2),
                       (v.shape[2] * 2 + 1, v.shape[3] * 2 - 1)):
            for op, call in (("nearest", lambda t: ops.upsample_nearest2d(t, (ho, wo))),
                             ("nearest_exact", lambda t: ops.upsample_nearest_exact2d(t, (ho, wo))),
                             ("bilinear", lambda t: ops.upsample_bilinear2d(t, (ho, wo), align))):
                want = call(dense)
                got, count = _launches(ops, lambda: call(v))
                assert torch.equal(got, want), (name, op, ho, wo)
                if op != "bilinear":
                    pitched = wo == 2 * v.shape[3] and ho % v.shape[2] == 0 and v.stride(3) == 1
                    assert (count == 1) == pitched, (name, op, ho, wo, count)
                elif name == "channel slice" and wo == 2 * v.shape[3]:
                    # 16-byte aligned pitches: the 2x-width kernel reads the view in place (the dense call's launches)
                    _, dense_count = _launches(ops, lambda: call(dense))
                    assert count == dense_count, (name, op, ho, wo, count, dense_count)
    # an up-sample written straight into a channel slice of a larger buffer (up-sample + concatenate)
    x = base[:, :5, :8, :16].contiguous()
    cat = torch.full((3, 12, 16, 32), 7.0, dtype=dtype, device=dev)
    for op, call in (("nearest", lambda t, o: ops.upsample_nearest2d(t, (16, 32), out=o)),
                     ("bilinear", lambda t, o: ops.upsample_bilinear2d(t, (16, 32), align, out=o))):
        for src in (x, base[:, :5, 3:11, 16:32]):   # dense input, cropped input
            cat.fill_(7.0)
            _, dense_count = _launches(ops, lambda: call(src.contiguous(), None))
            _, count = _launches(ops, lambda: call(src, cat[:, 4:9]))
            if op == "nearest":
                assert count == 1, count
            elif src is x:   # the 2x-width bilinear kernel takes the output's pitches: the launches of a dense call
                assert count == dense_count, (count, dense_count)
            assert torch.equal(cat[:, 4:9], call(src.contiguous(), None)), op
            assert float((cat[:, :4] - 7.0).abs().max()) == 0.0 and float((cat[:, 9:] - 7.0).abs().max()) == 0.0
    # down-scaling into a view with a W stride of 2
    v = base[:, :, 1:19, 2:30]
    out_base = torch.zeros((3, 6, 7, 22), dtype=dtype, device=dev)
    out = out_base[:, :, :, ::2]
    ops.upsample_bilinear2d(v, (7, 11), align, out=out)
    assert torch.equal(out, ops.upsample_bilinear2d(v.contiguous(), (7, 11), align))
    assert float(out_base[:, :, :, 1::2].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_nearest_backward_between_pitched_views(ops, dev, dtype):
    """grad_output as a channel slice of the gradient of a concatenation, grad_input as a crop of a larger buffer:
    the 2x pool kernel with pitches gives the bits of the dense call in one launch."""
    cat_grad = torch.randn((3, 12, 16, 32), generator=gen(93)).to(dtype).to(dev)
    g = cat_grad[:, 4:9]
    assert not g.is_contiguous()
    for exact, call in ((False, ops.upsample_nearest2d_backward), (True, ops.upsample_nearest_exact2d_backward)):
        for hin in (8, 4):   # H factors 2 and 4
            want = call(g.contiguous(), (16, 32), (3, 5, hin, 16))
            got, count = _launches(ops, lambda: call(g, (16, 32), (3, 5, hin, 16)))
            assert torch.equal(got, want) and count == 1, (exact, hin, count)
            buf = torch.full((3, 5, hin + 2, 24), 5.0, dtype=dtype, device=dev)
            _, count = _launches(ops, lambda: call(g, (16, 32), (3, 5, hin, 16), out=buf[:, :, 1:1 + hin, 8:24]))
            assert count == 1
            assert torch.equal(buf[:, :, 1:1 + hin, 8:24], want)
            assert float((buf[:, :, 0] - 5.0).abs().max()) == 0.0 and float((buf[:, :, :, :8] - 5.0).abs().max()) == 0.0
    # a ragged size goes through the staging copies and still matches
    want = ops.upsample_nearest2d_backward(g.contiguous(), (16, 32), (3, 5, 7, 13))
    assert torch.equal(ops.upsample_nearest2d_backward(g, (16, 32), (3, 5, 7, 13)), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_bilinear_backward_reads_a_pitched_grad_output(ops, dev, dtype):
    """grad_output as a channel slice of the gradient of a concatenation feeds the 2x gather kernel through its
    pitches: the bits and the launch count of the dense call."""
    cat_grad = torch.randn((2, 12, 32, 64), generator=gen(94)).to(dtype).to(dev)
    g = cat_grad[:, 4:9]
    assert not g.is_contiguous()
    want, dense_count = _launches(ops, lambda: ops.upsample_bilinear2d_backward(g.contiguous(), (32, 64), (2, 5, 16, 32), False))
    got, count = _launches(ops, lambda: ops.upsample_bilinear2d_backward(g, (32, 64), (2, 5, 16, 32), False))
    assert torch.equal(got, want)
    assert count == dense_count, (count, dense_count)
    # other scales and a strided grad_input go through the staging copies and still match
    want = ops.upsample_bilinear2d_backward(g.contiguous(), (32, 64), (2, 5, 13, 20), True)
    assert torch.equal(ops.upsample_bilinear2d_backward(g, (32, 64), (2, 5, 13, 20), True), want)
