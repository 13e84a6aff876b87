"""Generates tests/golden/resample_golden.npz.

Run where a checkout of the reference is present and pass its path as the first argument; the resulting file is
committed, so the tests themselves never need the reference.

Sources of the golden outputs (the reference stores no golden vectors; its tests create them at test time):
  * GridSampler2D forward: the reference's own Python golden, image/grid_sampler2_d/tests/assets/golden.py
    (GridSampler2DComposeSpec.golden), imported and called here.
  * every other op: the PyTorch-CPU calls the reference's kernel-UT generators and ST executors make
    (e.g. image/upsample_bilinear2d/tests/ut/op_kernel/upsample_bilinear2d_data/gen_data.py:37-39,
    image/grid_sample/tests/st/aclnnGridSampler2D/executor_aclnnGridSampler2D.py:48-52): fp32 compute,
    torch.nn.functional.interpolate / grid_sample and their autograd backward.
  * the fixed inputs of the reference's example clients (bilinear {0..7} 1x1x4x2 -> 8x4 align_corners=true,
    image/upsample_bilinear2d/examples/test_aclnn_upsample_bilinear2d.cpp:89-92; grid-sampler backward input
    {0..39} (1,1,5,8) with a 3x3 grid on {-1,0,1}, image/grid_sampler2_d_grad/examples/
    test_aclnn_grid_sampler2_d_backward.cpp:107-109), with outputs computed by the same torch calls.
Inputs are seeded (the reference's generators are not).
"""
import importlib.util
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py <path of the reference checkout>")
REF = sys.argv[1]
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "resample_golden.npz")


def load_ref_golden():
    path = os.path.join(REF, "image/grid_sampler2_d/tests/assets/golden.py")
    spec = importlib.util.spec_from_file_location("ref_grid_sampler_golden", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.GridSampler2DComposeSpec


def main():
    torch.manual_seed(20240611)
    torch.set_num_threads(1)
    data = {}
    meta = []

    def interp_case(name, mode, shape, out, align, scales, antialias=False):
        x = torch.randn(shape, dtype=torch.float32)
        kw = {}
        if mode != "nearest":
            kw["align_corners"] = align
        if antialias:
            kw["antialias"] = True
        if scales is None:
            kw["size"] = out
        else:
            kw["scale_factor"] = scales
            kw["recompute_scale_factor"] = False
        xg = x.clone().requires_grad_(True)
        y = F.interpolate(xg, mode=mode, **kw)
        assert tuple(y.shape[2:]) == tuple(out), (name, y.shape, out)
        g = torch.randn_like(y)
        y.backward(g)
        data[name + ".x"] = x.numpy()
        data[name + ".y"] = y.detach().numpy()
        data[name + ".g"] = g.numpy()
        data[name + ".gx"] = xg.grad.numpy()
        meta.append((name, mode, shape, out, align, scales))

    # nearest
    interp_case("nearest.up2", "nearest", (2, 3, 7, 9), (14, 18), False, None)
    interp_case("nearest.odd", "nearest", (2, 3, 7, 9), (15, 20), False, None)
    interp_case("nearest.down", "nearest", (1, 2, 16, 16), (5, 7), False, None)
    interp_case("nearest.scales", "nearest", (1, 2, 5, 6), (12, 16), False, (2.5, 2.7))
    # bilinear
    for align in (False, True):
        tag = "ac" if align else "hp"
        interp_case(f"bilinear.up2.{tag}", "bilinear", (2, 3, 7, 9), (14, 18), align, None)
        interp_case(f"bilinear.odd.{tag}", "bilinear", (2, 3, 7, 9), (15, 20), align, None)
        interp_case(f"bilinear.down.{tag}", "bilinear", (1, 2, 16, 16), (5, 7), align, None)
    interp_case("bilinear.cfg1like", "bilinear", (1, 3, 16, 16), (32, 32), False, None)
    interp_case("bilinear.scales", "bilinear", (1, 2, 8, 8), (16, 16), False, (2.0, 2.0))
    # bicubic anti-aliased
    for align in (False, True):
        tag = "ac" if align else "hp"
        interp_case(f"bicubic_aa.down.{tag}", "bicubic", (1, 2, 32, 40), (7, 9), align, None, antialias=True)
        interp_case(f"bicubic_aa.up.{tag}", "bicubic", (1, 2, 6, 7), (13, 15), align, None, antialias=True)
    interp_case("bicubic_aa.cfg3like", "bicubic", (1, 1, 64, 64), (14, 14), False, None, antialias=True)

    # example client of the reference (bilinear, align_corners=true)
    x = torch.arange(8, dtype=torch.float32).reshape(1, 1, 4, 2)
    data["example.bilinear.x"] = x.numpy()
    data["example.bilinear.y"] = F.interpolate(x, size=(8, 4), mode="bilinear", align_corners=True).numpy()

    # grid sampler: forward through the reference's own golden.py, backward through torch autograd
    spec = load_ref_golden()
    modes = ["bilinear", "nearest", "bicubic"]
    pads = ["zeros", "border", "reflection"]
    for mi, mode in enumerate(modes):
        for pi, pad in enumerate(pads):
            for align in (False, True):
                name = f"grid.{mode}.{pad}.{'ac' if align else 'hp'}"
                x = torch.randn((2, 3, 6, 7), dtype=torch.float32)
                grid = torch.rand((2, 5, 4, 2), dtype=torch.float32) * 2.6 - 1.3
                y = spec.golden(x.numpy(), grid.numpy(), interpolation_mode=mi, padding_mode=pi, align_corners=align)
                data[name + ".x"] = x.numpy()
                data[name + ".grid"] = grid.numpy()
                data[name + ".y"] = y
                if mode != "bicubic":
                    xg = x.clone().requires_grad_(True)
                    gg = grid.clone().requires_grad_(True)
                    yy = F.grid_sample(xg, gg, mode=mode, padding_mode=pad, align_corners=align)
                    g = torch.randn_like(yy)
                    yy.backward(g)
                    data[name + ".g"] = g.numpy()
                    data[name + ".gx"] = xg.grad.numpy()
                    data[name + ".ggrid"] = gg.grad.numpy()
    # example client of the reference (grid sampler backward)
    x = torch.arange(40, dtype=torch.float32).reshape(1, 1, 5, 8)
    lattice = torch.tensor([-1.0, 0.0, 1.0])
    gy, gx = torch.meshgrid(lattice, lattice, indexing="ij")
    grid = torch.stack([gx, gy], dim=-1).reshape(1, 3, 3, 2).contiguous()
    xg = x.clone().requires_grad_(True)
    gg = grid.clone().requires_grad_(True)
    yy = F.grid_sample(xg, gg, mode="bilinear", padding_mode="zeros", align_corners=False)
    g = torch.ones_like(yy)
    yy.backward(g)
    data["example.grid.x"] = x.numpy()
    data["example.grid.grid"] = grid.numpy()
    data["example.grid.y"] = yy.detach().numpy()
    data["example.grid.gx"] = xg.grad.numpy()
    data["example.grid.ggrid"] = gg.grad.numpy()

    data["meta.interp"] = np.array([repr(m) for m in meta])
    data["meta.torch_version"] = np.array(torch.__version__)
    np.savez_compressed(OUT, **data)
    print("wrote", OUT, os.path.getsize(OUT), "bytes,", len(data), "arrays")


if __name__ == "__main__":
    main()
