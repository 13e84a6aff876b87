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

A second file, tests/golden/atk_replay.npz, replays the reference's own test inputs:
  * a seeded slice of every ST case matrix of the hot-path APIs (image/*/tests/st/aclnn*/atk_aclnn*.json: ~200
    cases per API with shapes, dtypes, attributes and value distributions), with the torch CPU call of the matching
    executor_aclnn*.py (16-bit inputs up-cast to fp32, computed in fp32; backward cases with grad_output = ones as
    the executors do, and with a seeded random grad_output beside it). N and C are cut to at most 2 and 3 (they do
    not enter the arithmetic) and cases whose planes are too large for a small fixture are skipped;
  * the reference's kernel-UT generator for UpsampleBilinear2d, imported and run
    (image/upsample_bilinear2d/tests/ut/op_kernel/upsample_bilinear2d_data/gen_data.py, numpy seeded from outside).
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


# ---------------------------------------------------------------------------------------------------------------
# replay of the reference's ST case matrices and kernel-UT generators
# ---------------------------------------------------------------------------------------------------------------
ATK = {
    # api: (json path, kind)
    "UpsampleNearest2d": ("image/resize_nearest_neighbor_v2/tests/st/aclnnUpsampleNearest2d/atk_aclnnUpsampleNearest2d.json", "interp_fwd"),
    "UpsampleNearest2dBackward": ("image/upsample_nearest2d_grad/tests/st/aclnnUpsampleNearest2dBackward/atk_aclnnUpsampleNearest2dBackward.json", "interp_bwd"),
    "UpsampleBilinear2d": ("image/upsample_bilinear2d/tests/st/aclnnUpsampleBilinear2d/atk_aclnnUpsampleBilinear2d.json", "interp_fwd"),
    "UpsampleBilinear2dBackward": ("image/resize_bilinear_v2_grad/tests/st/aclnnUpsampleBilinear2dBackward/atk_aclnnUpsampleBilinear2dBackward.json", "interp_bwd"),
    "UpsampleBilinear2dBackwardV2": ("image/upsample_bilinear2d_grad/tests/st/aclnnUpsampleBilinear2dBackwardV2/atk_aclnnUpsampleBilinear2dBackwardV2.json", "interp_bwd"),
    "UpsampleBicubic2dAA": ("image/upsample_bicubic2d_aa/tests/st/aclnnUpsampleBicubic2dAA/atk_aclnnUpsampleBicubic2dAA.json", "interp_fwd"),
    "UpsampleBicubic2dAAGrad": ("image/upsample_bicubic2d_aa_grad/tests/st/aclnnUpsampleBicubic2dAAGrad/atk_aclnnUpsampleBicubic2dAAGrad.json", "interp_bwd"),
    "GridSampler2D": ("image/grid_sample/tests/st/aclnnGridSampler2D/atk_aclnnGridSampler2D.json", "grid_fwd"),
    "GridSampler2DBackward": ("image/grid_sampler2_d_grad/tests/st/aclnnGridSampler2DBackward/atk_aclnnGridSampler2DBackward.json", "grid_bwd"),
    "UpsampleBicubic2d": ("image/upsample_bicubic2d/tests/st/aclnnUpsampleBicubic2d/atk_aclnnUpsampleBicubic2d.json", "interp_fwd"),
    "UpsampleBicubic2dBackward": ("image/upsample_bicubic2d_grad/tests/st/aclnnUpsampleBicubic2dBackward/atk_aclnnUpsampleBicubic2dBackward.json", "interp_bwd"),
    "UpsampleBilinear2dAA": ("image/upsample_bilinear2d_aa/tests/st/aclnnUpsampleBilinear2dAA/atk_aclnnUpsampleBilinear2dAA.json", "interp_fwd"),
    "UpsampleBilinear2dAABackward": ("image/upsample_bilinear2d_aa_backward/tests/st/aclnnUpsampleBilinear2dAABackward/atk_aclnnUpsampleBilinear2dAABackward.json", "interp_bwd"),
    "UpsampleNearestExact2d": ("image/upsample_nearest/tests/st/aclnnUpsampleNearestExact2d/atk_aclnnUpsampleNearestExact2d.json", "interp_fwd"),
    "UpsampleNearestExact2dBackward": ("image/upsample_nearest_exact2d_grad/tests/st/aclnnUpsampleNearestExact2dBackward/atk_aclnnUpsampleNearestExact2dBackward.json", "interp_bwd"),
    "UpsampleNearest3d": ("image/upsample_nearest3d/tests/st/aclnnUpsampleNearest3d/atk_aclnnUpsampleNearest3d.json", "interp3_fwd"),
    "UpsampleNearest3dBackward": ("image/upsample_nearest3d_grad/tests/st/aclnnUpsampleNearest3dBackward/atk_aclnnUpsampleNearest3dBackward.json", "interp3_bwd"),
    "UpsampleNearestExact3d": ("image/upsample_nearest_exact3d/tests/st/aclnnUpsampleNearestExact3d/atk_aclnnUpsampleNearestExact3d.json", "interp3_fwd"),
    "UpsampleNearestExact3dBackward": ("image/upsample_nearest_exact3d_grad/tests/st/aclnnUpsampleNearestExact3dBackward/atk_aclnnUpsampleNearestExact3dBackward.json", "interp3_bwd"),
    "UpsampleTrilinear3d": ("image/resize_upsample_trilinear/tests/st/aclnnUpsampleTrilinear3d/atk_aclnnUpsampleTrilinear3d.json", "interp3_fwd"),
    "UpsampleTrilinear3dBackward": ("image/upsample_trilinear3d_backward/tests/st/aclnnUpsampleTrilinear3dBackward/atk_aclnnUpsampleTrilinear3dBackward.json", "interp3_bwd"),
    "GridSampler3D": ("image/grid_sample/tests/st/aclnnGridSampler3D/atk_aclnnGridSampler3D.json", "grid3_fwd"),
    "GridSampler3DBackward": ("image/grid_sampler3_d_grad/tests/st/aclnnGridSampler3DBackward/atk_aclnnGridSampler3DBackward.json", "grid3_bwd"),
}
SCALE_FACTOR_APIS = ("UpsampleBilinear2dAA", "UpsampleBilinear2dAABackward", "UpsampleNearestExact2d",
                     "UpsampleNearestExact2dBackward")
TORCH_DT = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}
CASES_PER_API = 20
MAX_PLANE = 1000   # H * W of any tensor of a kept case
MAX_VOLUME = 9000  # D * H * W of any tensor of a kept 3-D case (those keep one batch entry and two channels)


def case_fields(case):
    """Flattens the `inputs` list of an ATK case into {name: value}: tensors -> (dtype, shape, range), int arrays ->
    list, scalar attributes -> value."""
    out = {}
    for inp in case["inputs"]:
        if isinstance(inp, list):
            if inp:
                out[inp[0]["name"]] = [i.get("range_values") for i in inp]
        elif inp.get("type") == "tensor":
            out[inp["name"]] = ("tensor", inp["dtype"], inp["shape"], inp["range_values"])
        else:
            out[inp["name"]] = inp.get("range_values")
    return out


def draw(rng, shape, spec, dtype):
    """A seeded tensor with the case's value distribution, rounded to the case's dtype and returned as fp32."""
    if isinstance(spec, dict):  # {"name": "nd", "mean": [lo, hi], "std": [lo, hi]}
        mean, std = rng.uniform(*spec["mean"]), rng.uniform(*spec["std"])
        a = rng.normal(mean, std, size=shape)
    elif isinstance(spec, list) and len(spec) == 2 and all(isinstance(v, (int, float)) for v in spec):
        a = rng.uniform(spec[0], spec[1], size=shape)
    else:
        return None  # special-value cases (inf / nan fills) are covered by the parity tests' own cases
    return torch.from_numpy(a.astype(np.float32)).to(dtype).float()


def as_bool(v):
    return v if isinstance(v, bool) else str(v).lower() == "true"


def replay_atk(data, index):
    import json
    for api, (rel, kind) in ATK.items():
        cases = json.load(open(os.path.join(REF, rel)))
        kept = 0
        for case in cases:
            if kept >= (12 if kind.startswith("interp3") else CASES_PER_API):
                break
            f = case_fields(case)
            rng = np.random.default_rng(7000 + 1000 * list(ATK).index(api) + int(case["id"]))
            name = f"atk.{api}.{case['id']}"
            if kind in ("interp3_fwd", "interp3_bwd"):
                # the executors call interpolate(input, size=size, mode=mode[, align_corners]); the scales are 0
                _, dt, shape, spec = f["input"]
                if dt not in TORCH_DT or len(shape) != 5 or "size" not in f:
                    continue
                n, c, d, h, w = min(shape[0], 1), min(shape[1], 2), shape[2], shape[3], shape[4]
                od, oh, ow = f["size"]
                if min(n, c, d, h, w, od, oh, ow) < 1 or d * h * w > MAX_VOLUME or od * oh * ow > MAX_VOLUME:
                    continue
                x = draw(rng, (n, c, d, h, w), spec, TORCH_DT[dt])
                if x is None:
                    continue
                mode = f.get("mode", "nearest")
                kw = {"size": (od, oh, ow), "mode": mode}
                if mode == "trilinear":
                    kw["align_corners"] = as_bool(f.get("align_corners", False))
                xg = x.clone().requires_grad_(kind == "interp3_bwd")
                y = F.interpolate(xg, **kw)
                data[name + ".x"] = x.numpy()
                meta = {"api": api, "dtype": dt, "shape": [n, c, d, h, w], "size": [od, oh, ow], "mode": mode,
                        "align": kw.get("align_corners", False)}
                if kind == "interp3_fwd":
                    data[name + ".y"] = y.detach().numpy()
                else:
                    (gx_ones,) = torch.autograd.grad(y, xg, torch.ones_like(y), retain_graph=True)
                    g = torch.from_numpy(rng.standard_normal(tuple(y.shape)).astype(np.float32)).to(TORCH_DT[dt]).float()
                    (gx_rand,) = torch.autograd.grad(y, xg, g)
                    data[name + ".g"] = g.numpy()
                    data[name + ".gx_ones"] = gx_ones.numpy()
                    data[name + ".gx"] = gx_rand.numpy()
                index.append(meta | {"name": name})
                kept += 1
            elif kind in ("grid3_fwd", "grid3_bwd"):
                _, dt, ishape, ispec = f["input"]
                _, _, gshape, gspec = f["grid"]
                if dt not in TORCH_DT or len(ishape) != 5:
                    continue
                n, c = min(ishape[0], 2), min(ishape[1], 3)
                d, h, w = ishape[2], ishape[3], ishape[4]
                # samples are independent of each other: a large grid is cut to its first 8 x 8 x 8 samples
                do, ho, wo = min(gshape[1], 8), min(gshape[2], 8), min(gshape[3], 8)
                if min(n, c, d, h, w, do, ho, wo) < 1 or d * h * w > MAX_VOLUME:
                    continue
                x = draw(rng, (n, c, d, h, w), ispec, TORCH_DT[dt])
                grid = draw(rng, (n, do, ho, wo, 3), gspec, TORCH_DT[dt])
                if x is None or grid is None:
                    continue
                mode = int(f.get("mode", 0))
                pad = int(f.get("padding_mode", 0))
                align = as_bool(f.get("align_corners", False))
                if mode > 1:
                    continue
                data[name + ".x"] = x.numpy()
                data[name + ".grid"] = grid.numpy()
                meta = {"api": api, "dtype": dt, "mode": mode, "pad": pad, "align": align, "name": name}
                if kind == "grid3_fwd":
                    data[name + ".y"] = F.grid_sample(x, grid, mode=["bilinear", "nearest"][mode],
                                                      padding_mode=["zeros", "border", "reflection"][pad],
                                                      align_corners=align).numpy()
                else:
                    _, _, _, gospec = f["gradOutput"]
                    go = draw(rng, (n, c, do, ho, wo), gospec, TORCH_DT[dt])
                    if go is None:
                        continue
                    gi, gg = torch.ops.aten.grid_sampler_3d_backward(go, x, grid, mode, pad, align, [True, True])
                    data[name + ".g"] = go.numpy()
                    data[name + ".gx"] = gi.numpy()
                    data[name + ".ggrid"] = gg.numpy()
                index.append(meta)
                kept += 1
            elif kind in ("interp_fwd", "interp_bwd"):
                _, dt, shape, spec = f["input"]
                # cases given by scale_factor are replayed for the APIs added after the first fixture was cut (a
                # change for the others would reshuffle their kept cases)
                by_factor = "size" not in f and "scale_factor" in f and api in SCALE_FACTOR_APIS
                if dt not in TORCH_DT or len(shape) != 4 or ("size" not in f and not by_factor):
                    continue
                n, c, h, w = min(shape[0], 2), min(shape[1], 3), shape[2], shape[3]
                if by_factor:
                    sf = [float(v) for v in f["scale_factor"]]
                    oh, ow = int(np.floor(h * sf[0])), int(np.floor(w * sf[1]))
                else:
                    oh, ow = f["size"]
                if min(n, c, h, w, oh, ow) < 1 or h * w > MAX_PLANE or oh * ow > MAX_PLANE:
                    continue
                x = draw(rng, (n, c, h, w), spec, TORCH_DT[dt])
                if x is None:
                    continue
                mode = f.get("mode", "nearest")
                kw = {"scale_factor": sf, "recompute_scale_factor": False, "mode": mode} if by_factor else {
                    "size": (oh, ow), "mode": mode}
                if mode not in ("nearest", "nearest-exact"):
                    kw["align_corners"] = as_bool(f.get("align_corners", False))
                if as_bool(f.get("antialias", False)):
                    kw["antialias"] = True
                xg = x.clone().requires_grad_(kind == "interp_bwd")
                y = F.interpolate(xg, **kw)
                assert tuple(y.shape[2:]) == (oh, ow)
                data[name + ".x"] = x.numpy() if dt == "fp32" else x.to(torch.float16 if dt == "fp16" else torch.float32).numpy()
                meta = {"api": api, "dtype": dt, "shape": [n, c, h, w], "size": [oh, ow], "mode": mode,
                        "align": kw.get("align_corners", False), "aa": kw.get("antialias", False)}
                if by_factor:
                    meta["scales"] = sf
                if kind == "interp_fwd":
                    data[name + ".y"] = y.detach().numpy()
                else:
                    # grad_output = ones, as executor_aclnnUpsampleBilinear2dBackwardV2.py:82-83, and a seeded random one
                    (gx_ones,) = torch.autograd.grad(y, xg, torch.ones_like(y), retain_graph=True)
                    g = torch.from_numpy(rng.standard_normal(tuple(y.shape)).astype(np.float32)).to(TORCH_DT[dt]).float()
                    (gx_rand,) = torch.autograd.grad(y, xg, g)
                    data[name + ".g"] = g.numpy()
                    data[name + ".gx_ones"] = gx_ones.numpy()
                    data[name + ".gx"] = gx_rand.numpy()
                index.append(meta | {"name": name})
                kept += 1
            else:
                _, dt, ishape, ispec = f["input"]
                _, _, gshape, gspec = f["grid"]
                if dt not in TORCH_DT or len(ishape) != 4:
                    continue
                n, c, h, w = min(ishape[0], 2), min(ishape[1], 3), ishape[2], ishape[3]
                # samples are independent of each other: a large grid is cut to its first 24 x 24 samples
                ho, wo = min(gshape[1], 24), min(gshape[2], 24)
                if min(n, c, h, w, ho, wo) < 1 or h * w > MAX_PLANE + 100:
                    continue
                x = draw(rng, (n, c, h, w), ispec, TORCH_DT[dt])
                grid = draw(rng, (n, ho, wo, 2), gspec, TORCH_DT[dt])
                if x is None or grid is None:
                    continue
                mode = int(f.get("mode", f.get("interpolationMode", 0)))
                pad = int(f.get("padding_mode", f.get("paddingMode", 0)))
                align = as_bool(f.get("align_corners", f.get("alignCorners", False)))
                data[name + ".x"] = x.numpy()
                data[name + ".grid"] = grid.numpy()
                meta = {"api": api, "dtype": dt, "mode": mode, "pad": pad, "align": align, "name": name}
                if kind == "grid_fwd":
                    data[name + ".y"] = F.grid_sample(x, grid, mode=["bilinear", "nearest", "bicubic"][mode],
                                                      padding_mode=["zeros", "border", "reflection"][pad],
                                                      align_corners=align).numpy()
                else:
                    _, _, _, gospec = f["gradOutput"]
                    go = draw(rng, (n, c, ho, wo), gospec, TORCH_DT[dt])
                    gi, gg = torch.ops.aten.grid_sampler_2d_backward(go, x, grid, mode, pad, align, [True, True])
                    data[name + ".g"] = go.numpy()
                    data[name + ".gx"] = gi.numpy()
                    data[name + ".ggrid"] = gg.numpy()
                index.append(meta)
                kept += 1
        print(f"{api}: {kept} cases of {len(cases)}")


def replay_gen_data(data, index):
    """Runs the reference's kernel-UT generator of UpsampleBilinear2d in a scratch directory (it writes the input and
    the torch golden as .bin files) and stores what it wrote."""
    import runpy
    import tempfile
    gen = os.path.join(REF, "image/upsample_bilinear2d/tests/ut/op_kernel/upsample_bilinear2d_data/gen_data.py")
    mod = runpy.run_path(gen)
    cwd = os.getcwd()
    for i, (shape, size) in enumerate([("(1,1,4,4)", "(16,16)"), ("(2,3,9,7)", "(5,20)"), ("(1,2,16,16)", "(32,32)")]):
        with tempfile.TemporaryDirectory() as tmp:
            os.chdir(tmp)
            try:
                np.random.seed(4242 + i)
                mod["gen_data_and_golden"](shape, size, f"case{i}", "float32")
                x = np.fromfile(f"case{i}_float32_input_upsample_bilinear2d.bin", dtype=np.float32)
                y = np.fromfile(f"case{i}_float32_golden_upsample_bilinear2d.bin", dtype=np.float32)
            finally:
                os.chdir(cwd)
        ishape, osize = eval(shape), eval(size)
        name = f"gen_data.UpsampleBilinear2d.{i}"
        data[name + ".x"] = x.reshape(ishape)
        data[name + ".y"] = y.reshape(ishape[:2] + osize)
        index.append({"api": "UpsampleBilinear2d", "dtype": "fp32", "shape": list(ishape), "size": list(osize),
                      "mode": "bilinear", "align": False, "aa": False, "name": name})


def main_replay():
    import json
    torch.set_num_threads(1)
    data, index = {}, []
    replay_atk(data, index)
    replay_gen_data(data, index)
    data["index"] = np.array(json.dumps(index))
    data["meta.torch_version"] = np.array(torch.__version__)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "atk_replay.npz")
    np.savez_compressed(out, **data)
    print("wrote", out, os.path.getsize(out), "bytes,", len(index), "cases")


if __name__ == "__main__":
    if len(sys.argv) > 2 and sys.argv[2] == "replay":
        main_replay()
    else:
        main()
