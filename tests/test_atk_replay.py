"""Replay of the reference's own test inputs (tests/golden/atk_replay.npz, made by tests/golden/make_golden.py
<reference> replay): a seeded slice of the ST case matrices of twenty-three APIs plus the kernel-UT generator of
UpsampleBilinear2d, each with the torch CPU golden that the reference's executors compute.

The CPU half holds the oracle to these goldens, the GPU half the library (through the C ABI). The bar is the one the
reference's kernel UTs use against the same torch goldens (compare_data.py: fp32 rtol 1e-4; 16-bit 1e-2 relative),
with the absolute term scaled by the magnitude of the case (the matrices draw values from N(mean in [-100, 100],
std in [1, 25])); every case's largest error relative to that magnitude is collected and the worst per API is
reported in the assertion message of a failing case and by `pytest -s`."""
import json
import os

import numpy as np
import pytest
import torch

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "atk_replay.npz"))
INDEX = json.loads(str(GOLD["index"]))
DT = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}
APIS = sorted({m["api"] for m in INDEX})


def bar(dtype):
    return {"fp32": 1e-4, "fp16": 2.0 ** -9, "bf16": 2.0 ** -6}[dtype]


def rel_err(got, ref):
    """Largest |got - ref| relative to the magnitude of the case (so that results that cancel to nearly zero are
    measured against the values they were formed from)."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    fin = np.isfinite(ref)
    assert np.array_equal(np.isfinite(got), fin)
    if not fin.any():
        return 0.0
    scale = max(float(np.abs(ref[fin]).max()), 1.0)
    return float(np.abs(got[fin] - ref[fin]).max()) / scale


def run_case(m, backend, oracle):
    """backend: "oracle" (numpy in, numpy out) or the ops module (GPU). Returns {output name: (got, golden)}."""
    name, api = m["name"], m["api"]
    x = GOLD[name + ".x"].astype(np.float32)
    dt = DT[m["dtype"]]
    out = {}
    gpu = backend != "oracle"
    dev = torch.device("cuda:0") if gpu else None
    t = (lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dt).to(dev)) if gpu else None
    back = lambda y: y.float().cpu().numpy()  # noqa: E731
    rnd = lambda a: torch.from_numpy(a).to(dt).float().numpy()  # noqa: E731  (the oracle's result in the case's dtype)
    if api.endswith("3d") or api.endswith("3dBackward"):
        size, align, shape = tuple(m["size"]), bool(m["align"]), tuple(m["shape"])
        exact, tri = "Exact" in api, "Trilinear" in api
        if not api.endswith("Backward"):
            if tri:
                got = back(backend.upsample_trilinear3d(t(x), size, align)) if gpu else rnd(
                    oracle.trilinear3d_fwd(x, size, align))
            else:
                got = back(backend.upsample_nearest3d(t(x), size, exact=exact)) if gpu else rnd(
                    oracle.nearest3d_fwd(x, size, exact=exact))
            out["y"] = (got, GOLD[name + ".y"])
        else:
            for gname, gold in (("ones", "gx_ones"), ("rand", "gx")):
                g = np.ones((shape[0], shape[1]) + size, np.float32) if gname == "ones" else GOLD[name + ".g"]
                if tri:
                    got = back(backend.upsample_trilinear3d_backward(t(g), size, shape, align)) if gpu else rnd(
                        oracle.trilinear3d_bwd(g, shape[2:], align))
                else:
                    got = back(backend.upsample_nearest3d_backward(t(g), size, shape, exact=exact)) if gpu else rnd(
                        oracle.nearest3d_bwd(g, shape[2:], exact=exact))
                out[gold] = (got, GOLD[name + "." + gold])
    elif api.startswith("GridSampler3D"):
        grid = GOLD[name + ".grid"].astype(np.float32)
        mode, pad, align = m["mode"], m["pad"], bool(m["align"])
        if api == "GridSampler3D":
            if not gpu and mode != 0:
                return out  # the oracle states the reference's bilinear kernel only; nearest is held on the GPU half
            got = back(backend.grid_sampler3d(t(x), t(grid), mode, pad, align)) if gpu else rnd(
                oracle.grid_sampler3d_fwd(x, grid, pad, align))
            out["y"] = (got, GOLD[name + ".y"])
        else:
            g = GOLD[name + ".g"]
            if gpu:
                gi, gg = backend.grid_sampler3d_backward(t(g), t(x), t(grid), mode, pad, align)
                gi, gg = back(gi), back(gg)
            else:
                gi, gg = oracle.grid_sampler3d_bwd(g, x, grid, mode, pad, align)
                gi, gg = rnd(gi), rnd(gg)
            out["gx"] = (gi, GOLD[name + ".gx"])
            out["ggrid"] = (gg, GOLD[name + ".ggrid"])
    elif api.startswith("Upsample"):
        size, align, shape = tuple(m["size"]), bool(m["align"]), tuple(m["shape"])
        scales = tuple(m.get("scales", (0.0, 0.0)))
        if api == "UpsampleNearest2d":
            got = back(backend.upsample_nearest2d(t(x), size)) if gpu else rnd(oracle.nearest2d_fwd(x, size))
            out["y"] = (got, GOLD[name + ".y"])
        elif api == "UpsampleBilinear2d":
            got = back(backend.upsample_bilinear2d(t(x), size, align)) if gpu else rnd(oracle.bilinear2d_fwd(x, size, align))
            out["y"] = (got, GOLD[name + ".y"])
        elif api == "UpsampleBicubic2d":
            got = back(backend.upsample_bicubic2d(t(x), size, align)) if gpu else rnd(oracle.bicubic2d_fwd(x, size, align))
            out["y"] = (got, GOLD[name + ".y"])
        elif api == "UpsampleNearestExact2d":
            got = back(backend.upsample_nearest_exact2d(t(x), size, scales=scales)) if gpu else rnd(
                oracle.nearest_exact2d_fwd(x, size, scales))
            out["y"] = (got, GOLD[name + ".y"])
        elif api == "UpsampleBilinear2dAA":
            got = back(backend.upsample_bilinear2d_aa(t(x), size, align, scales)) if gpu else rnd(
                oracle.bilinear_aa_fwd(x, size, align, scales))
            out["y"] = (got, GOLD[name + ".y"])
        elif api == "UpsampleBicubic2dAA":
            got = back(backend.upsample_bicubic2d_aa(t(x), size, align)) if gpu else rnd(oracle.bicubic_aa_fwd(x, size, align))
            out["y"] = (got, GOLD[name + ".y"])
        else:
            for gname, gold in (("ones", "gx_ones"), ("rand", "gx")):
                g = np.ones((shape[0], shape[1]) + size, np.float32) if gname == "ones" else GOLD[name + ".g"]
                if api == "UpsampleNearest2dBackward":
                    got = back(backend.upsample_nearest2d_backward(t(g), size, shape)) if gpu else rnd(
                        oracle.nearest2d_bwd(g, shape[2:]))
                elif api.startswith("UpsampleBilinear2dBackward"):
                    v2 = api.endswith("V2")
                    got = back(backend.upsample_bilinear2d_backward(t(g), size, shape, align, v2=v2)) if gpu else rnd(
                        oracle.bilinear2d_bwd(g, shape[2:], align, definition="dispatch"))
                elif api == "UpsampleNearestExact2dBackward":
                    got = back(backend.upsample_nearest_exact2d_backward(t(g), size, shape, scales)) if gpu else rnd(
                        oracle.nearest_exact2d_bwd(g, shape[2:], scales))
                elif api == "UpsampleBilinear2dAABackward":
                    got = back(backend.upsample_bilinear2d_aa_backward(t(g), size, shape, align, scales)) if gpu else rnd(
                        oracle.bilinear_aa_bwd(g, shape[2:], align, scales))
                elif api == "UpsampleBicubic2dBackward":
                    got = back(backend.upsample_bicubic2d_backward(t(g), size, shape, align)) if gpu else rnd(
                        oracle.bicubic2d_bwd(g, shape[2:], align, definition="dispatch"))
                else:
                    got = back(backend.upsample_bicubic2d_aa_grad(t(g), size, shape, align)) if gpu else rnd(
                        oracle.bicubic_aa_bwd(g, shape[2:], align))
                out[gold] = (got, GOLD[name + "." + gold])
    else:
        grid = GOLD[name + ".grid"].astype(np.float32)
        mode, pad, align = m["mode"], m["pad"], bool(m["align"])
        if api == "GridSampler2D":
            got = back(backend.grid_sampler2d(t(x), t(grid), mode, pad, align)) if gpu else rnd(
                oracle.grid_sampler2d_fwd(x, grid, mode, pad, align))
            out["y"] = (got, GOLD[name + ".y"])
        else:
            g = GOLD[name + ".g"]
            if gpu:
                gi, gg = backend.grid_sampler2d_backward(t(g), t(x), t(grid), mode, pad, align)
                gi, gg = back(gi), back(gg)
            else:
                gi, gg = oracle.grid_sampler2d_bwd(g, x, grid, mode, pad, align)
                gi, gg = rnd(gi), rnd(gg)
            out["gx"] = (gi, GOLD[name + ".gx"])
            out["ggrid"] = (gg, GOLD[name + ".ggrid"])
    return out


def check_api(api, backend, oracle):
    worst, count = {}, 0
    for m in INDEX:
        if m["api"] != api:
            continue
        count += 1
        for key, (got, gold) in run_case(m, backend, oracle).items():
            ref = torch.from_numpy(np.asarray(gold, np.float32)).to(DT[m["dtype"]]).float().numpy()
            e = rel_err(got, ref)
            worst[(m["dtype"], key)] = max(worst.get((m["dtype"], key), 0.0), e)
            assert e <= bar(m["dtype"]), f"{m['name']} {key}: {e:.3e} of the case's magnitude (bar {bar(m['dtype']):.1e})"
    assert count >= 3
    print(f"{api}: {count} cases, largest error relative to the case's magnitude per (dtype, output): "
          + ", ".join(f"{k}={v:.2e}" for k, v in sorted(worst.items())))


@pytest.mark.parametrize("api", APIS)
def test_oracle_against_replayed_reference_tests(oracle, api):
    check_api(api, "oracle", oracle)


@pytest.mark.gpu
@pytest.mark.parametrize("api", APIS)
def test_library_against_replayed_reference_tests(ops, oracle, dev, api):
    check_api(api, ops, oracle)
