#!/usr/bin/env python
"""Benchmark of the resampling hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload default|cfg2|cfg3|cfg4|cfg4bf16|cfg5|adj2|adj3|adj4|adj5|all]
                    [--batch-div D] [--impl reference]

One "step" is one pass of every operator of the workload over one batch of seeded synthetic input, called
through the library's C ABI (two-phase aclnn calls). The default workload is the FPN-style up-sampling case
(UpsampleNearest2d and UpsampleBilinear2d, forward and backward, fp16 NCHW 32x256x56x56 -> 112x112).

Printed JSON (one line, rank 0):
  value      effective HBM GB/s = algorithmic bytes of all operators of a step / device time, inputs resident in
             HBM, summed over ranks (every rank runs the same per-GPU workload: weak scaling, no collective);
  e2e        the same metric with HOST buffers: pinned host -> device copies of the step's inputs and device ->
             host copies of its results inside the timed region;
  roofline   the operator with the largest share of the step: algorithmic bytes per launch / average launch
             duration (CUDA events on the launching stream) against the measured HBM copy peak;
  ops        the same figures for every operator of the workload;
  cpu_baseline  the CPU oracle (the reference's kernel arithmetic restated in C++/OpenMP) on a bounded sample, and
             beside it the torch CPU operators the reference's own test scripts use as their golden, same sample;
  other_workloads  (default run, one GPU) the same per-operator figures for the other benchmark configurations,
             fewer steps each, every one with its own clock record;
  box_sweep  the box-sweep configuration (bilinear bf16 NHWC N=512 plus grid sampler fp32 N=256) split evenly along N over the ranks (strong scaling): box time = slowest rank,
             efficiency = T(1) / (G * T(G)) with T(1) measured in the same run on the whole batch.

Timing: CUDA events on the launching stream, max over ranks; every step works on a different one of several
buffer sets whose total exceeds the L2 capacity, so no operator finds its input in L2.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_FALLBACK_BYTES = 126 * 1024 * 1024


def l2_bytes(torch=None, dev=None):
    """L2 capacity of the device (cudaDeviceProp::l2CacheSize); the B200 figure when no device is visible."""
    try:
        if torch is not None and torch.cuda.is_available():
            return int(torch.cuda.get_device_properties(dev if dev is not None else 0).L2_cache_size)
    except Exception:  # noqa: BLE001 - any failure means "no device to ask"
        pass
    return L2_FALLBACK_BYTES


def buffer_sets(set_bytes, l2, wanted=0):
    """How many buffer sets a workload rotates: enough to exceed L2 four times, at least 3, at most 16."""
    return min(wanted or max(3, -(-4 * l2 // set_bytes)), 16)


def l2_note(nsets, set_bytes, l2):
    return (f"rotating {nsets} buffer sets of {set_bytes / 1e6:.0f} MB ({nsets * set_bytes / 1e6:.0f} MB > "
            f"{l2 / 1e6:.0f} MB L2): each step's inputs come from HBM")


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs, STREAM-style copy)"
    return 6650.0, "fallback (6.65 TB/s: no MEASURED_PEAKS.json beside this file)"


# ncu dram__bytes_read.sum + dram__bytes_write.sum per launch of the main kernel of each operator, copied from the
# captures summarised under profiles/ (None = not captured). These are constants from earlier profiler runs, not
# measurements of this run: every row that carries one also names the summary it comes from (TRAFFIC_SOURCE).
TRAFFIC_SOURCE = {"cfg2": "profiles/cfg2_fpn_upsample_kernels_ncu.md", "cfg3": "profiles/cfg3_bicubic_aa_kernels_ncu.md",
                  "cfg4": "profiles/cfg4_grid_sampler_kernels_ncu.md", "cfg5": "profiles/cfg5_box_sweep_kernels_ncu.md"}
NCU_TRAFFIC = {
    ("cfg2", "UpsampleNearest2d"): 201.0e6, ("cfg2", "UpsampleBilinear2d"): 206.1e6,
    ("cfg2", "UpsampleNearest2dBackward"): 242.2e6, ("cfg2", "UpsampleBilinear2dBackward"): 208.0e6,
    ("cfg3", "UpsampleBicubic2dAA"): 864.1e6, ("cfg3", "UpsampleBicubic2dAAGrad"): 785.0e6,
    ("cfg4", "GridSampler2D"): 278.9e6, ("cfg4", "GridSampler2DBackward[atomic]"): 394.8e6,
    ("cfg4", "GridSampler2DBackward[deterministic]"): 326.8e6 + 447.9e6,  # gather + grad_grid kernels
    ("cfg5", "UpsampleBilinear2d[NHWC bf16]"): 5311.5e6, ("cfg5", "GridSampler2D[affine fp32]"): 2252.0e6,
}
# rows whose figure comes from a single-kernel capture of a reduced batch, scaled by the batch divisor
TRAFFIC_SOURCE_OP = {("cfg2", "UpsampleBilinear2dBackward"): "profiles/cfg2_bilinear_backward_kernel_ncu.md",
                     ("cfg5", "GridSampler2D[affine fp32]"): "profiles/cfg5_grid_sampler_window_kernel_ncu.md"}


# ---------------------------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------------------------
class Op:
    def __init__(self, name, run, algo_bytes, pixels, inputs, outputs):
        self.name = name          # operator name
        self.run = run            # run(buffers) -> None, enqueues on the current stream
        self.algo_bytes = algo_bytes
        self.pixels = pixels      # output spatial locations N*Hout*Wout
        self.inputs = inputs      # names of buffers copied host -> device in the e2e arm
        self.outputs = outputs    # names of buffers copied device -> host in the e2e arm


def nbytes(t):
    return t.numel() * t.element_size()


def make_workload(name, ops, torch, dev, batch_div=1, shard=None):
    """Returns (make_buffers(gen) -> dict of tensors on the generator's device, [Op], config dict).
    batch_div: the batch divided by this (small cases for profiler captures). shard = (world, rank): cfg5 only, the
    rank's share of the box-level batch (contiguous split along N)."""
    ws = ops.Workspace(dev) if ops is not None else None  # None: only the description is wanted
    # one workspace per operator for workloads whose operators are independent of each other: they may then run on
    # parallel branches of the step graph
    wss = [ws] + [ops.Workspace(dev) for _ in range(5)] if ops is not None else [None] * 6

    if name == "cfg2":
        n, c, hi, wi, ho, wo = 32 // batch_div, 256, 56, 56, 112, 112
        dt = torch.float16

        def buffers(gen):
            return {
                "x": torch.randn((n, c, hi, wi), generator=gen, device=gen.device).to(dt),
                "go": torch.randn((n, c, ho, wo), generator=gen, device=gen.device).to(dt),
                "y_nearest": torch.empty((n, c, ho, wo), dtype=dt, device=gen.device),
                "y_bilinear": torch.empty((n, c, ho, wo), dtype=dt, device=gen.device),
                "gi_nearest": torch.empty((n, c, hi, wi), dtype=dt, device=gen.device),
                "gi_bilinear": torch.empty((n, c, hi, wi), dtype=dt, device=gen.device),
            }
        small, big = n * c * hi * wi * 2, n * c * ho * wo * 2
        oplist = [
            Op("UpsampleNearest2d", lambda b: ops.upsample_nearest2d(b["x"], (ho, wo), out=b["y_nearest"], workspace=wss[0]),
               small + big, n * ho * wo, ["x"], ["y_nearest"]),
            Op("UpsampleBilinear2d", lambda b: ops.upsample_bilinear2d(b["x"], (ho, wo), False, scales=(2.0, 2.0),
                                                                       out=b["y_bilinear"], workspace=wss[1]),
               small + big, n * ho * wo, ["x"], ["y_bilinear"]),
            Op("UpsampleNearest2dBackward", lambda b: ops.upsample_nearest2d_backward(
                b["go"], (ho, wo), (n, c, hi, wi), scales=(2.0, 2.0), out=b["gi_nearest"], workspace=wss[2]),
               small + big, n * ho * wo, ["go"], ["gi_nearest"]),
            Op("UpsampleBilinear2dBackward", lambda b: ops.upsample_bilinear2d_backward(
                b["go"], (ho, wo), (n, c, hi, wi), False, scales=(2.0, 2.0), out=b["gi_bilinear"], workspace=wss[3]),
               small + big, n * ho * wo, ["go"], ["gi_bilinear"]),
        ]
        cfg = {"workload": "FPN-style upsampling: UpsampleNearest2d + UpsampleBilinear2d forward and backward, fp16 "
                           f"NCHW N={n} C=256 56x56 -> 112x112 (scale 2.0), align_corners=false",
               "dtype": "f16"}
        return buffers, oplist, cfg

    if name == "cfg3":
        n, c, hi, wi, ho, wo = 64 // batch_div, 3, 1024, 1024, 224, 224
        dt = torch.float32

        def buffers(gen):
            return {
                "x": (torch.randint(0, 256, (n, c, hi, wi), generator=gen, device=gen.device).to(dt) / 255.0),
                "go": torch.randn((n, c, ho, wo), generator=gen, device=gen.device),
                "y": torch.empty((n, c, ho, wo), dtype=dt, device=gen.device),
                "gi": torch.empty((n, c, hi, wi), dtype=dt, device=gen.device),
            }
        big, small = n * c * hi * wi * 4, n * c * ho * wo * 4
        oplist = [
            Op("UpsampleBicubic2dAA", lambda b: ops.upsample_bicubic2d_aa(b["x"], (ho, wo), False, out=b["y"], workspace=wss[0]),
               small + big, n * ho * wo, ["x"], ["y"]),
            Op("UpsampleBicubic2dAAGrad", lambda b: ops.upsample_bicubic2d_aa_grad(
                b["go"], (ho, wo), (n, c, hi, wi), False, out=b["gi"], workspace=wss[1]),
               small + big, n * ho * wo, ["go"], ["gi"]),
        ]
        cfg = {"workload": f"UpsampleBicubic2dAA forward and backward, fp32 NCHW N={n} C=3 1024x1024 -> 224x224 "
                           "(a = -0.5, support 2*scale), align_corners=false", "dtype": "f32"}
        return buffers, oplist, cfg

    if name in ("cfg4", "cfg4bf16", "cfg4affine"):
        # cfg4affine: the cfg4 shapes with smooth grids (random rotation / scale / shift, as in cfg5) instead of
        # uniform-random sample positions; not one of the benchmark configurations, it separates the cost of the random
        # access pattern from the cost of the kernels
        n, c, hi, wi, ho, wo = 16 // batch_div, 256, 64, 64, 128, 128
        dt = torch.bfloat16 if name == "cfg4bf16" else torch.float32
        es = 2 if name == "cfg4bf16" else 4

        def make_grid(gen):
            if name != "cfg4affine":
                return torch.rand((n, ho, wo, 2), generator=gen, device=gen.device) * 2.2 - 1.1
            import math
            phi = (torch.rand(n, generator=gen, device=gen.device) * 60 - 30) * math.pi / 180
            sc = torch.rand(n, generator=gen, device=gen.device) * 0.4 + 0.8
            t = torch.rand((n, 2), generator=gen, device=gen.device) * 0.2 - 0.1
            theta = torch.stack([torch.stack([sc * torch.cos(phi), -sc * torch.sin(phi), t[:, 0]], 1),
                                 torch.stack([sc * torch.sin(phi), sc * torch.cos(phi), t[:, 1]], 1)], 1)
            return torch.nn.functional.affine_grid(theta, (n, c, ho, wo), align_corners=False).contiguous()

        def buffers(gen):
            return {
                "x": torch.randn((n, c, hi, wi), generator=gen, device=gen.device).to(dt),
                "grid": make_grid(gen).to(dt),
                "go": torch.randn((n, c, ho, wo), generator=gen, device=gen.device).to(dt),
                "y": torch.empty((n, c, ho, wo), dtype=dt, device=gen.device),
                "gi": torch.empty((n, c, hi, wi), dtype=dt, device=gen.device),
                "ggrid": torch.empty((n, ho, wo, 2), dtype=dt, device=gen.device),
            }
        xin, gr, out = n * c * hi * wi * es, n * ho * wo * 2 * es, n * c * ho * wo * es

        def bwd(det):
            def run(b):
                ops.set_deterministic(det)
                try:
                    ops.grid_sampler2d_backward(b["go"], b["x"], b["grid"], 0, 0, False, input_grad=b["gi"],
                                                grid_grad=b["ggrid"], workspace=ws)
                finally:
                    ops.set_deterministic(False)
            return run
        oplist = [
            Op("GridSampler2D", lambda b: ops.grid_sampler2d(b["x"], b["grid"], 0, 0, False, out=b["y"], workspace=ws),
               xin + gr + out, n * ho * wo, ["x", "grid"], ["y"]),
            Op("GridSampler2DBackward[atomic]", bwd(False), out + xin + gr + xin + gr, n * ho * wo,
               ["go", "x", "grid"], ["gi", "ggrid"]),
            Op("GridSampler2DBackward[deterministic]", bwd(True), out + xin + gr + xin + gr, n * ho * wo,
               ["go", "x", "grid"], ["gi", "ggrid"]),
        ]
        cfg = {"workload": f"GridSampler2D forward + backward, bilinear/zeros/align_corners=false, {str(dt)[6:]} N={n} "
                           "C=256 64x64, grid 128x128 " +
                           ("random affine (rotation +-30 deg, scale 0.8-1.2, shift +-0.1)" if name == "cfg4affine"
                            else "uniform[-1.1,1.1]"), "dtype": "f32" if es == 4 else "bf16"}
        return buffers, oplist, cfg

    if name == "adj2":
        # the operators next to the path at the cfg2 shapes: UpsampleNearestExact2d and UpsampleBicubic2d
        n, c, hi, wi, ho, wo = 32 // batch_div, 256, 56, 56, 112, 112
        dt = torch.float16

        def buffers(gen):
            return {
                "x": torch.randn((n, c, hi, wi), generator=gen, device=gen.device).to(dt),
                "go": torch.randn((n, c, ho, wo), generator=gen, device=gen.device).to(dt),
                "y_exact": torch.empty((n, c, ho, wo), dtype=dt, device=gen.device),
                "y_bicubic": torch.empty((n, c, ho, wo), dtype=dt, device=gen.device),
                "gi_exact": torch.empty((n, c, hi, wi), dtype=dt, device=gen.device),
                "gi_bicubic": torch.empty((n, c, hi, wi), dtype=dt, device=gen.device),
                "y_bicubic_ac": torch.empty((n, c, ho, wo), dtype=dt, device=gen.device),
                "gi_bicubic_ac": torch.empty((n, c, hi, wi), dtype=dt, device=gen.device),
            }
        small, big = n * c * hi * wi * 2, n * c * ho * wo * 2
        oplist = [
            Op("UpsampleNearestExact2d", lambda b: ops.upsample_nearest_exact2d(b["x"], (ho, wo), out=b["y_exact"],
                                                                                workspace=wss[0]),
               small + big, n * ho * wo, ["x"], ["y_exact"]),
            Op("UpsampleBicubic2d", lambda b: ops.upsample_bicubic2d(b["x"], (ho, wo), False, out=b["y_bicubic"],
                                                                     workspace=wss[1]),
               small + big, n * ho * wo, ["x"], ["y_bicubic"]),
            Op("UpsampleNearestExact2dBackward", lambda b: ops.upsample_nearest_exact2d_backward(
                b["go"], (ho, wo), (n, c, hi, wi), out=b["gi_exact"], workspace=wss[2]),
               small + big, n * ho * wo, ["go"], ["gi_exact"]),
            Op("UpsampleBicubic2dBackward", lambda b: ops.upsample_bicubic2d_backward(
                b["go"], (ho, wo), (n, c, hi, wi), False, out=b["gi_bicubic"], workspace=wss[3]),
               small + big, n * ho * wo, ["go"], ["gi_bicubic"]),
            # the same tensors with align_corners=true: the scale is 55 / 111, so these two run the general kernels
            # (the calls above are exactly 2x and run the kernels of that scale)
            Op("UpsampleBicubic2d[align_corners]", lambda b: ops.upsample_bicubic2d(
                b["x"], (ho, wo), True, out=b["y_bicubic_ac"], workspace=wss[4]),
               small + big, n * ho * wo, ["x"], ["y_bicubic_ac"]),
            Op("UpsampleBicubic2dBackward[align_corners]", lambda b: ops.upsample_bicubic2d_backward(
                b["go"], (ho, wo), (n, c, hi, wi), True, out=b["gi_bicubic_ac"], workspace=wss[5]),
               small + big, n * ho * wo, ["go"], ["gi_bicubic_ac"]),
        ]
        cfg = {"workload": "operators next to the path at the FPN shapes: UpsampleNearestExact2d + UpsampleBicubic2d "
                           f"forward and backward, fp16 NCHW N={n} C=256 56x56 -> 112x112, align_corners=false; "
                           "UpsampleBicubic2d again with align_corners=true",
               "dtype": "f16"}
        return buffers, oplist, cfg

    if name == "adj3":
        # UpsampleBilinear2dAA at the cfg3 shapes
        n, c, hi, wi, ho, wo = 64 // batch_div, 3, 1024, 1024, 224, 224
        dt = torch.float32

        def buffers(gen):
            return {
                "x": (torch.randint(0, 256, (n, c, hi, wi), generator=gen, device=gen.device).to(dt) / 255.0),
                "go": torch.randn((n, c, ho, wo), generator=gen, device=gen.device),
                "y": torch.empty((n, c, ho, wo), dtype=dt, device=gen.device),
                "gi": torch.empty((n, c, hi, wi), dtype=dt, device=gen.device),
            }
        big, small = n * c * hi * wi * 4, n * c * ho * wo * 4
        oplist = [
            Op("UpsampleBilinear2dAA", lambda b: ops.upsample_bilinear2d_aa(b["x"], (ho, wo), False, out=b["y"],
                                                                            workspace=wss[0]),
               small + big, n * ho * wo, ["x"], ["y"]),
            Op("UpsampleBilinear2dAABackward", lambda b: ops.upsample_bilinear2d_aa_backward(
                b["go"], (ho, wo), (n, c, hi, wi), False, out=b["gi"], workspace=wss[1]),
               small + big, n * ho * wo, ["go"], ["gi"]),
        ]
        cfg = {"workload": f"UpsampleBilinear2dAA forward and backward, fp32 NCHW N={n} C=3 1024x1024 -> 224x224 "
                           "(triangle filter, support = scale), align_corners=false", "dtype": "f32"}
        return buffers, oplist, cfg

    if name == "adj4":
        # the 3-D siblings of the up-samplers on a volumetric feature map: nearest and trilinear, both directions
        n, c, di, hi, wi, do, ho, wo = max(2 // batch_div, 1), 32, 32, 56, 56, 64, 112, 112
        dt = torch.float16

        def buffers(gen):
            return {
                "x": torch.randn((n, c, di, hi, wi), generator=gen, device=gen.device).to(dt),
                "go": torch.randn((n, c, do, ho, wo), generator=gen, device=gen.device).to(dt),
                "y_nearest": torch.empty((n, c, do, ho, wo), dtype=dt, device=gen.device),
                "y_trilinear": torch.empty((n, c, do, ho, wo), dtype=dt, device=gen.device),
                "gi_nearest": torch.empty((n, c, di, hi, wi), dtype=dt, device=gen.device),
                "gi_trilinear": torch.empty((n, c, di, hi, wi), dtype=dt, device=gen.device),
            }
        small, big = n * c * di * hi * wi * 2, n * c * do * ho * wo * 2
        oplist = [
            Op("UpsampleNearest3d", lambda b: ops.upsample_nearest3d(b["x"], (do, ho, wo), out=b["y_nearest"],
                                                                      workspace=wss[0]),
               small + big, n * do * ho * wo, ["x"], ["y_nearest"]),
            Op("UpsampleTrilinear3d", lambda b: ops.upsample_trilinear3d(b["x"], (do, ho, wo), False,
                                                                          out=b["y_trilinear"], workspace=wss[1]),
               small + big, n * do * ho * wo, ["x"], ["y_trilinear"]),
            Op("UpsampleNearest3dBackward", lambda b: ops.upsample_nearest3d_backward(
                b["go"], (do, ho, wo), (n, c, di, hi, wi), out=b["gi_nearest"], workspace=wss[2]),
               small + big, n * do * ho * wo, ["go"], ["gi_nearest"]),
            Op("UpsampleTrilinear3dBackward", lambda b: ops.upsample_trilinear3d_backward(
                b["go"], (do, ho, wo), (n, c, di, hi, wi), False, out=b["gi_trilinear"], workspace=wss[3]),
               small + big, n * do * ho * wo, ["go"], ["gi_trilinear"]),
        ]
        cfg = {"workload": "3-D siblings on a volumetric feature map: UpsampleNearest3d + UpsampleTrilinear3d forward "
                           f"and backward, fp16 NCDHW N={n} C=32 32x56x56 -> 64x112x112, align_corners=false",
               "dtype": "f16"}
        return buffers, oplist, cfg

    if name == "adj5":
        # GridSampler3D forward and backward, trilinear taps, uniform-random sample positions
        n, c, di, hi, wi, do, ho, wo = max(2 // batch_div, 1), 32, 32, 64, 64, 32, 64, 64
        dt = torch.float32

        def buffers(gen):
            return {
                "x": torch.randn((n, c, di, hi, wi), generator=gen, device=gen.device),
                "grid": torch.rand((n, do, ho, wo, 3), generator=gen, device=gen.device) * 2.2 - 1.1,
                "go": torch.randn((n, c, do, ho, wo), generator=gen, device=gen.device),
                "y": torch.empty((n, c, do, ho, wo), dtype=dt, device=gen.device),
                "gi": torch.empty((n, c, di, hi, wi), dtype=dt, device=gen.device),
                "ggrid": torch.empty((n, do, ho, wo, 3), dtype=dt, device=gen.device),
                # the same tensors channels-last (NDHWC)
                "x_cl": torch.randn((n, di, hi, wi, c), generator=gen, device=gen.device),
                "go_cl": torch.randn((n, do, ho, wo, c), generator=gen, device=gen.device),
                "y_cl": torch.empty((n, do, ho, wo, c), dtype=dt, device=gen.device),
                "gi_cl": torch.empty((n, di, hi, wi, c), dtype=dt, device=gen.device),
                "ggrid_cl": torch.empty((n, do, ho, wo, 3), dtype=dt, device=gen.device),
            }
        xin, gr, out = n * c * di * hi * wi * 4, n * do * ho * wo * 3 * 4, n * c * do * ho * wo * 4
        oplist = [
            Op("GridSampler3D", lambda b: ops.grid_sampler3d(b["x"], b["grid"], 0, 0, False, out=b["y"],
                                                              workspace=wss[0]),
               xin + gr + out, n * do * ho * wo, ["x", "grid"], ["y"]),
            Op("GridSampler3DBackward", lambda b: ops.grid_sampler3d_backward(
                b["go"], b["x"], b["grid"], 0, 0, False, input_grad=b["gi"], grid_grad=b["ggrid"], workspace=wss[1]),
               out + xin + gr + xin + gr, n * do * ho * wo, ["go", "x", "grid"], ["gi", "ggrid"]),
            Op("GridSampler3D[NDHWC]", lambda b: ops.grid_sampler3d(b["x_cl"], b["grid"], 0, 0, False, fmt="NDHWC",
                                                                     out=b["y_cl"], workspace=wss[2]),
               xin + gr + out, n * do * ho * wo, ["x_cl", "grid"], ["y_cl"]),
            Op("GridSampler3DBackward[NDHWC]", lambda b: ops.grid_sampler3d_backward(
                b["go_cl"], b["x_cl"], b["grid"], 0, 0, False, fmt="NDHWC", input_grad=b["gi_cl"],
                grid_grad=b["ggrid_cl"], workspace=wss[3]),
               out + xin + gr + xin + gr, n * do * ho * wo, ["go_cl", "x_cl", "grid"], ["gi_cl", "ggrid_cl"]),
        ]
        cfg = {"workload": f"GridSampler3D forward + backward, bilinear/zeros/align_corners=false, fp32 NCDHW and NDHWC N={n} "
                           "C=32 32x64x64, grid 32x64x64 uniform[-1.1,1.1]", "dtype": "f32"}
        return buffers, oplist, cfg

    if name == "cfg5":
        import math
        n, c, hi, wi, ho, wo = 512 // batch_div, 256, 64, 64, 128, 128
        n2, c2, h2 = 256 // batch_div, 128, 96
        total = (n, n2)
        if shard is not None:
            from opscv_b200 import sharding
            b, e = sharding.shard_range(n, *shard)
            b2, e2 = sharding.shard_range(n2, *shard)
            n, n2 = e - b, e2 - b2

        def buffers(gen):
            dv = gen.device
            phi = (torch.rand(n2, generator=gen, device=dv) * 60 - 30) * math.pi / 180
            s = torch.rand(n2, generator=gen, device=dv) * 0.4 + 0.8
            t = torch.rand((n2, 2), generator=gen, device=dv) * 0.2 - 0.1
            theta = torch.stack([torch.stack([s * torch.cos(phi), -s * torch.sin(phi), t[:, 0]], 1),
                                 torch.stack([s * torch.sin(phi), s * torch.cos(phi), t[:, 1]], 1)], 1)
            grid = torch.nn.functional.affine_grid(theta, (n2, c2, h2, h2), align_corners=False)
            return {
                "x": torch.randn((n, hi, wi, c), generator=gen, device=dv).to(torch.bfloat16),
                "y": torch.empty((n, ho, wo, c), dtype=torch.bfloat16, device=dv),
                "gx": torch.randn((n2, c2, h2, h2), generator=gen, device=dv), "grid": grid.contiguous(),
                "gy": torch.empty((n2, c2, h2, h2), device=dv),
            }
        oplist = [
            Op("UpsampleBilinear2d[NHWC bf16]", lambda b: ops.upsample_bilinear2d(b["x"], (ho, wo), False, "NHWC",
                                                                                  out=b["y"], workspace=wss[0]),
               n * c * (hi * wi + ho * wo) * 2, n * ho * wo, ["x"], ["y"]),
            Op("GridSampler2D[affine fp32]", lambda b: ops.grid_sampler2d(b["gx"], b["grid"], 0, 0, False, out=b["gy"],
                                                                         workspace=wss[1]),
               n2 * c2 * h2 * h2 * 4 * 2 + n2 * h2 * h2 * 2 * 4, n2 * h2 * h2, ["gx", "grid"], ["gy"]),
        ]
        cfg = {"workload": f"box sweep: UpsampleBilinear2d bf16 NHWC N={n} C=256 64x64 -> 128x128 + GridSampler2D "
                           f"fp32 N={n2} C=128 96x96 affine grids" +
                           (f" (this rank's share of N={total[0]} / N={total[1]})" if shard is not None else ""),
               "dtype": "bf16/f32", "images": [n, n2]}
        return buffers, oplist, cfg
    raise ValueError(name)


# ---------------------------------------------------------------------------------------------------------------
# CUDA graphs through the runtime API (torch's graph wrapper adds a small fill kernel of its own to every replay,
# which would sit inside the per-operator event brackets)
# ---------------------------------------------------------------------------------------------------------------
class RawGraph:
    _rt = None

    @classmethod
    def rt(cls):
        if cls._rt is None:
            cls._rt = ctypes.CDLL("libcudart.so.12")  # the runtime torch has already loaded
        return cls._rt

    @staticmethod
    def _check(code, what):
        if code != 0:
            raise RuntimeError(f"{what} failed with CUDA error {code}")

    def __init__(self, torch, capture_stream, fn):
        rt, h = self.rt(), ctypes.c_void_p(capture_stream.cuda_stream)
        graph, self.exec_ = ctypes.c_void_p(), ctypes.c_void_p()
        with torch.cuda.stream(capture_stream):
            self._check(rt.cudaStreamBeginCapture(h, 1), "cudaStreamBeginCapture")  # thread-local mode
            try:
                fn()
            finally:
                code = rt.cudaStreamEndCapture(h, ctypes.byref(graph))
            self._check(code, "cudaStreamEndCapture")
        self._check(rt.cudaGraphInstantiate(ctypes.byref(self.exec_), graph, ctypes.c_ulonglong(0)),
                    "cudaGraphInstantiate")
        rt.cudaGraphDestroy(graph)

    def replay(self, stream):
        self._check(self.rt().cudaGraphLaunch(self.exec_, ctypes.c_void_p(stream.cuda_stream)), "cudaGraphLaunch")

    def __del__(self):
        if getattr(self, "exec_", None):
            self.rt().cudaGraphExecDestroy(self.exec_)


# ---------------------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx = float(s[1])
            except ValueError:
                continue
            for nme, v in zip(names, s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nme)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------------
# CPU baseline (the oracle, timed; never part of the GPU path)
# ---------------------------------------------------------------------------------------------------------------
def cpu_baseline(workload, budget_s=12.0, torch_budget_s=6.0):
    """Times two CPU arms on a bounded sample of `workload` on the host cores: the oracle (the reference's kernel
    arithmetic restated in C++/OpenMP) and, beside it, the torch CPU operators that the reference's own test scripts
    compute their goldens with. Returns the JSON object (value = the oracle's figure)."""
    import numpy as np
    import torch
    import torch.nn.functional as F
    import oracle
    oracle.build()
    # all host cores this process may use, whatever OMP_NUM_THREADS a launcher (torchrun sets 1) exported
    threads = len(os.sched_getaffinity(0))
    oracle.set_num_threads(threads)
    cores = oracle.num_threads()
    torch.set_num_threads(threads)
    rng = np.random.default_rng(1234)
    if workload in ("cfg2", "all", "default"):
        n, c = 4, 256  # 1/8 of the batch of the GPU workload; planes are independent
        x = rng.standard_normal((n, c, 56, 56)).astype(np.float32)
        go = rng.standard_normal((n, c, 112, 112)).astype(np.float32)
        small, big = x.size * 2, go.size * 2  # bytes at the fp16 storage dtype of the GPU workload

        def run():
            oracle.nearest2d_fwd(x, (112, 112))
            oracle.bilinear2d_fwd(x, (112, 112), False, (2.0, 2.0))
            oracle.nearest2d_bwd(go, (56, 56), (2.0, 2.0))
            # the kernel the reference dispatches for this call, the same definition the parity tests hold the GPU to
            oracle.bilinear2d_bwd(go, (56, 56), False, (2.0, 2.0), definition="dispatch")
        xt, got = torch.from_numpy(x), torch.from_numpy(go)

        def run_torch():
            F.interpolate(xt, size=(112, 112), mode="nearest")
            F.interpolate(xt, size=(112, 112), mode="bilinear", align_corners=False)
            torch.ops.aten.upsample_nearest2d_backward(got, [112, 112], [n, c, 56, 56], 2.0, 2.0)
            torch.ops.aten.upsample_bilinear2d_backward(got, [112, 112], [n, c, 56, 56], False, 2.0, 2.0)
        algo = 4 * (small + big)
        sample = f"N={n} of 32 images (C={c}), all four operators, fp32 arithmetic"
    elif workload == "cfg3":
        x = rng.random((1, 3, 1024, 1024), dtype=np.float32)
        go = rng.standard_normal((1, 3, 224, 224)).astype(np.float32)

        def run():
            oracle.bicubic_aa_fwd(x, (224, 224))
            oracle.bicubic_aa_bwd(go, (1024, 1024), definition="scatter")
        xt, got = torch.from_numpy(x), torch.from_numpy(go)

        def run_torch():
            F.interpolate(xt, size=(224, 224), mode="bicubic", align_corners=False, antialias=True)
            torch.ops.aten._upsample_bicubic2d_aa_backward(got, [224, 224], [1, 3, 1024, 1024], False, None, None)
        algo = 2 * (x.size + go.size) * 4
        sample = "N=1 of 64 images, forward + backward (scatter definition)"
    elif workload == "adj2":
        n, c = 4, 256
        x = rng.standard_normal((n, c, 56, 56)).astype(np.float32)
        go = rng.standard_normal((n, c, 112, 112)).astype(np.float32)

        def run():
            oracle.nearest_exact2d_fwd(x, (112, 112))
            oracle.bicubic2d_fwd(x, (112, 112), False)
            oracle.nearest_exact2d_bwd(go, (56, 56))
            oracle.bicubic2d_bwd(go, (56, 56), False, definition="dispatch")
            oracle.bicubic2d_fwd(x, (112, 112), True)
            oracle.bicubic2d_bwd(go, (56, 56), True, definition="dispatch")
        xt, got = torch.from_numpy(x), torch.from_numpy(go)

        def run_torch():
            F.interpolate(xt, size=(112, 112), mode="nearest-exact")
            F.interpolate(xt, size=(112, 112), mode="bicubic", align_corners=False)
            torch.ops.aten._upsample_nearest_exact2d_backward(got, [112, 112], [n, c, 56, 56], None, None)
            torch.ops.aten.upsample_bicubic2d_backward(got, [112, 112], [n, c, 56, 56], False, None, None)
            F.interpolate(xt, size=(112, 112), mode="bicubic", align_corners=True)
            torch.ops.aten.upsample_bicubic2d_backward(got, [112, 112], [n, c, 56, 56], True, None, None)
        algo = 6 * (x.size + go.size) * 2
        sample = f"N={n} of 32 images (C={c}), all six operators, fp32 arithmetic"
    elif workload == "adj3":
        x = rng.random((1, 3, 1024, 1024), dtype=np.float32)
        go = rng.standard_normal((1, 3, 224, 224)).astype(np.float32)

        def run():
            oracle.bilinear_aa_fwd(x, (224, 224))
            oracle.bilinear_aa_bwd(go, (1024, 1024), definition="scatter")
        xt, got = torch.from_numpy(x), torch.from_numpy(go)

        def run_torch():
            F.interpolate(xt, size=(224, 224), mode="bilinear", align_corners=False, antialias=True)
            torch.ops.aten._upsample_bilinear2d_aa_backward(got, [224, 224], [1, 3, 1024, 1024], False, None, None)
        algo = 2 * (x.size + go.size) * 4
        sample = "N=1 of 64 images, forward + backward (scatter definition)"
    elif workload == "adj4":
        x = rng.standard_normal((1, 4, 32, 56, 56)).astype(np.float32)
        go = rng.standard_normal((1, 4, 64, 112, 112)).astype(np.float32)

        def run():
            oracle.nearest3d_fwd(x, (64, 112, 112))
            oracle.trilinear3d_fwd(x, (64, 112, 112), False)
            oracle.nearest3d_bwd(go, (32, 56, 56))
            oracle.trilinear3d_bwd(go, (32, 56, 56), False)
        xt, got = torch.from_numpy(x), torch.from_numpy(go)

        def run_torch():
            F.interpolate(xt, size=(64, 112, 112), mode="nearest")
            F.interpolate(xt, size=(64, 112, 112), mode="trilinear", align_corners=False)
            torch.ops.aten.upsample_nearest3d_backward(got, [64, 112, 112], [1, 4, 32, 56, 56], None, None, None)
            torch.ops.aten.upsample_trilinear3d_backward(got, [64, 112, 112], [1, 4, 32, 56, 56], False, None, None,
                                                         None)
        algo = 4 * (x.size + go.size) * 2
        sample = "N=1, C=4 of N=2, C=32, all four operators, fp32 arithmetic"
    elif workload == "adj5":
        x = rng.standard_normal((1, 8, 32, 64, 64)).astype(np.float32)
        grid = (rng.random((1, 32, 64, 64, 3), dtype=np.float32) * 2.2 - 1.1)
        go = rng.standard_normal((1, 8, 32, 64, 64)).astype(np.float32)

        def run():
            oracle.grid_sampler3d_fwd(x, grid)
            oracle.grid_sampler3d_bwd(go, x, grid)
        xt, gt, got = torch.from_numpy(x), torch.from_numpy(grid), torch.from_numpy(go)

        def run_torch():
            F.grid_sample(xt, gt, mode="bilinear", padding_mode="zeros", align_corners=False)
            torch.ops.aten.grid_sampler_3d_backward(got, xt, gt, 0, 0, False, [True, True])
        algo = ((x.size + grid.size + go.size) + (go.size + 2 * x.size + 2 * grid.size)) * 4
        sample = "N=1, C=8 of N=2, C=32, forward + backward"
    elif workload in ("cfg4", "cfg4bf16", "cfg4affine"):
        es = 4 if workload == "cfg4" else 2
        x = rng.standard_normal((1, 256, 64, 64)).astype(np.float32)
        grid = (rng.random((1, 128, 128, 2), dtype=np.float32) * 2.2 - 1.1)
        go = rng.standard_normal((1, 256, 128, 128)).astype(np.float32)

        def run():
            oracle.grid_sampler2d_fwd(x, grid)
            oracle.grid_sampler2d_bwd(go, x, grid)
        xt, gt, got = torch.from_numpy(x), torch.from_numpy(grid), torch.from_numpy(go)

        def run_torch():
            F.grid_sample(xt, gt, mode="bilinear", padding_mode="zeros", align_corners=False)
            torch.ops.aten.grid_sampler_2d_backward(got, xt, gt, 0, 0, False, [True, True])
        algo = ((x.size + grid.size + go.size) + (go.size + 2 * x.size + 2 * grid.size)) * es
        sample = "N=1 of 16 images, forward + backward"
    else:
        x = rng.standard_normal((4, 64, 64, 256)).astype(np.float32)
        gx = rng.standard_normal((2, 128, 96, 96)).astype(np.float32)
        grid = (rng.random((2, 96, 96, 2), dtype=np.float32) * 2 - 1)

        def run():
            oracle.bilinear2d_fwd(x, (128, 128), False, fmt=oracle.NHWC)
            oracle.grid_sampler2d_fwd(gx, grid)
        xt = torch.from_numpy(x).permute(0, 3, 1, 2)  # channels-last storage seen as NCHW
        gxt, gt = torch.from_numpy(gx), torch.from_numpy(grid)

        def run_torch():
            F.interpolate(xt, size=(128, 128), mode="bilinear", align_corners=False)
            F.grid_sample(gxt, gt, mode="bilinear", padding_mode="zeros", align_corners=False)
        algo = x.size * 5 * 2 + (gx.size * 2 + grid.size) * 4
        sample = "N=4 of 512 (bilinear NHWC) and N=2 of 256 (grid sampler)"

    def clock(fn, budget):
        fn()  # warm-up (page faults, thread pools)
        t0 = time.perf_counter()
        reps = 0
        while True:
            fn()
            reps += 1
            if (time.perf_counter() - t0 > budget and reps >= 3) or reps >= 5000:
                break
        return (time.perf_counter() - t0) / reps, reps
    dt, reps = clock(run, budget_s)
    out = {"value": algo / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
           "sample": sample + f"; {reps} repetitions, {dt * 1e3:.1f} ms each", "ms_per_sample": dt * 1e3}
    try:
        with torch.no_grad():
            tdt, treps = clock(run_torch, torch_budget_s)
        out["torch_cpu"] = {"value": algo / tdt / 1e9, "unit": "GB/s", "threads": torch.get_num_threads(),
                            "sample": f"same sample, torch {torch.__version__} CPU operators (interpolate / grid_sample "
                                      f"and their aten backward functions); {treps} repetitions, {tdt * 1e3:.1f} ms each"}
    except Exception as exc:  # noqa: BLE001 - the torch arm is a second opinion; the port's figure stands without it
        out["torch_cpu"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
    return out


# ---------------------------------------------------------------------------------------------------------------
L2_RULE = ("no L2 flush: consecutive steps rotate over several buffer sets whose total is at least four times the L2 "
           "capacity (cudaDeviceProp::l2CacheSize), so every step reads its inputs from HBM; sizes in l2_detail")


def arm_config(cfg):
    """The `config` object of a workload: the same keys and values in this library's arm and in the CPU reference
    arm, which runs a bounded sample of the same workload (the sample is described in a key of its own)."""
    return {"workload": cfg["workload"], "per_gpu_batch": "fixed (weak scaling)", "l2": L2_RULE}


METRIC = "effective HBM GB/s (algorithmic bytes / device time), all operators of the step"
OTHER_WORKLOADS = ["cfg3", "cfg4", "cfg4bf16", "cfg5", "adj2", "adj3", "adj4", "adj5"]
LAUNCH_NOTE = ("CUDA-graph replay of the aclnn second-phase calls: the timed steps replay one graph per buffer set holding "
               "all operators of the step (cfg2, cfg3, cfg5, adj2 - adj5: the independent operators of a step on parallel branches, "
               "each with its own workspace; cfg4: one after the other, the two backward modes write the same tensors); "
               "the per-operator times come from a separate pass: per-operator graphs launched back to back over all "
               "buffer sets between one pair of events")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="default",
                    help="default = cfg2 as the head line plus the other configurations with fewer steps")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-others", action="store_true", help="default workload: skip the other configurations")
    ap.add_argument("--no-box-sweep", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time eager calls instead of CUDA-graph replays")
    ap.add_argument("--serial-step", action="store_true",
                    help="step graph with the operators one after the other instead of on parallel branches")
    ap.add_argument("--sets", type=int, default=0, help="buffer sets to rotate (0 = enough to exceed L2 four times)")
    ap.add_argument("--batch-div", type=int, default=1,
                    help="divide every batch by this: small cases for profiler captures (not a benchmark number)")
    ap.add_argument("--other-steps", type=int, default=60, help="timed steps of each of the other configurations")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    head_name = "cfg2" if args.workload in ("default", "all") else args.workload

    if args.impl == "reference":
        # The reference's own implementation of this path needs the CANN toolkit (Ascend C kernels) and cannot be
        # built here; its arithmetic restated on the CPU (the oracle) stands in, on all host threads, and the torch
        # CPU operators its test scripts take their goldens from are timed beside it.
        if rank != 0:
            return
        base = cpu_baseline(head_name, budget_s=max(5.0, min(60.0, 2.0 * args.steps)))
        import torch
        cfg = make_workload(head_name, None, torch, None)[2]
        line = {
            "impl": "reference", "metric": METRIC,
            "value": base["value"], "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": base["ms_per_sample"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": cfg["dtype"], "data": "synthetic (seeded)",
            "config": arm_config(cfg),
            "sample": "each step is a bounded sample of the workload on the host CPU: " + base["sample"],
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample", "torch_cpu")},
            "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }
        print(json.dumps(line))
        return

    import torch
    import __graft_entry__ as entry
    ops = entry.load_package()
    ops.lib()  # fail loudly if the CUDA library is missing
    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    peak, peak_src = measured_peak()
    ctx = dict(args=args, ops=ops, torch=torch, dev=dev, dist=dist, world=world, rank=rank, peak=peak)
    head = run_workload(head_name, steps=args.steps, do_e2e=not args.no_e2e, host_data=True, **ctx)
    torch.cuda.empty_cache()
    others = {}
    if args.workload == "all" or (args.workload == "default" and world == 1 and not args.no_others):
        for wname in OTHER_WORKLOADS:
            others[wname] = run_workload(wname, steps=min(args.steps, args.other_steps), do_e2e=False, host_data=False,
                                         **ctx)
            torch.cuda.empty_cache()
    sweep = None
    if args.workload in ("default", "all") and not args.no_box_sweep and args.batch_div == 1:
        sweep = box_sweep(others.get("cfg5"), **ctx)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    line = {
        "metric": METRIC,
        "value": head["value"], "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": head["config"]["dtype"], "data": "synthetic (seeded torch.Generator)",
        "config": arm_config(head["config"]), "l2_detail": head["l2_note"],
        "launch": "eager aclnn calls" if args.no_graph else LAUNCH_NOTE,
        "mpix_per_s": head["mpix_per_s"], "pct_of_hbm_peak": head["value"] / (peak * world),
        "roofline": head["roofline"], "ops": head["ops"], "e2e": head["e2e"], "gpu_launches": head["gpu_launches"],
        "clocks": head["clocks"], "peak_source": peak_src,
    }
    if args.batch_div != 1:
        line["batch_div"] = args.batch_div
    if not args.no_cpu_baseline and world == 1:  # reported at N=1 only
        base = cpu_baseline(head_name)
        line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample", "torch_cpu")}
    if others:
        line["other_workloads"] = {k: {kk: v[kk] for kk in ("value", "ms_per_step", "steps", "mpix_per_s", "ops", "clocks",
                                                            "gpu_launches", "l2_note", "config")}
                                   for k, v in others.items()}
    if sweep is not None:
        line["box_sweep"] = sweep
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def box_sweep(cfg5_result, args, ops, torch, dev, dist, world, rank, peak):
    """The box-sweep configuration (bilinear bf16 NHWC N=512 plus grid sampler fp32 N=256) split evenly along N over the ranks (strong scaling, no collective): rank r owns the
    images sharding.shard_range(N, world, r) of both operators. T(1) is the same workload with the whole batch on one
    GPU, measured in this run (every rank times it on its own GPU; the slowest counts); efficiency = T(1) / (G * T(G)).
    With one rank the object just restates the cfg5 figures as the sweep's G = 1 point."""
    steps = min(args.steps, args.other_steps)
    ctx = dict(args=args, ops=ops, torch=torch, dev=dev, dist=dist, world=world, rank=rank, peak=peak)
    whole = cfg5_result or run_workload("cfg5", steps=steps, do_e2e=False, host_data=False, **ctx)
    torch.cuda.empty_cache()
    part = whole if world == 1 else run_workload("cfg5", steps=steps, do_e2e=False, host_data=False,
                                                 shard=(world, rank), **ctx)
    torch.cuda.empty_cache()
    n_b, n_g = 512, 256
    pixels = n_b * 128 * 128 + n_g * 96 * 96
    algo = sum(r["algorithmic_bytes"] for r in whole["ops"].values())
    t1, tg = whole["ms_per_step"], part["ms_per_step"]
    op_rows = {}
    for name, row in whole["ops"].items():
        g = part["ops"][name]
        op_rows[name] = {"ms_1gpu": row["ms"], "ms": g["ms"], "efficiency": row["ms"] / (world * g["ms"]),
                         "box_gb_per_s": row["algorithmic_bytes"] / (g["ms"] * 1e-3) / 1e9,
                         "frac_of_peak_per_gpu": row["algorithmic_bytes"] / world / (g["ms"] * 1e-3) / 1e9 / peak}
    return {"workload": f"UpsampleBilinear2d bf16 NHWC N={n_b} C=256 64x64 -> 128x128 + GridSampler2D fp32 N={n_g} C=128 "
                        "96x96 random affine grids, split evenly along N over the ranks (contiguous, rank-local "
                        "tensors, no collective)",
            "scaling": "strong", "n_gpus": world,
            "images_per_rank": [-(-n_b // world), -(-n_g // world)],
            "ms_per_step_1gpu": t1, "ms_per_step": tg, "efficiency": t1 / (world * tg),
            "box_gb_per_s": algo / (tg * 1e-3) / 1e9, "box_mpix_per_s": pixels / tg / 1e3,
            "pct_of_hbm_peak_per_gpu": algo / world / (tg * 1e-3) / 1e9 / peak,
            "steps": steps, "ops": op_rows, "clocks": part["clocks"]}


def run_workload(wname, args, ops, torch, dev, dist, world, rank, peak, steps, do_e2e, host_data, shard=None):
    """One workload on this rank's GPU. host_data: the seeded inputs are drawn on the CPU and copied in (needed by the
    end-to-end arm); otherwise they are drawn on the device from a seeded device generator (large configurations)."""
    make_buffers, oplist, cfg = make_workload(wname, ops, torch, dev, args.batch_div, shard)
    if host_data:
        host = make_buffers(torch.Generator().manual_seed(1234 + rank))
        set_bytes = sum(nbytes(t) for t in host.values())
    else:
        host = None
        first = make_buffers(torch.Generator(device=dev).manual_seed(1234 + rank))
        set_bytes = sum(nbytes(t) for t in first.values())
    l2 = l2_bytes(torch, dev)
    nsets = buffer_sets(set_bytes, l2, args.sets)
    if host_data:
        dsets = [{k: v.to(dev) for k, v in host.items()} for _ in range(nsets)]
    else:
        dsets = [first] + [{k: v.clone() for k, v in first.items()} for _ in range(nsets - 1)]
    note = l2_note(nsets, set_bytes, l2)
    stream = torch.cuda.current_stream(dev)

    def barrier():
        torch.cuda.synchronize(dev)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-resident arm --------------------------------------------------------------------------------
    # Eager warm-up (also grows the workspace to its final size), then every (operator, buffer set) pair is
    # captured once into a CUDA graph of its second-phase call; the timed loop replays the graphs, so that the
    # Python cost of building aclTensor handles does not leave the GPU idle between ~50 us kernels.
    for i in range(max(args.warmup, nsets)):
        for op in oplist:
            op.run(dsets[i % nsets])
    barrier()
    use_graph = not args.no_graph
    launches_per_step = 0
    step_graphs = None
    if use_graph:
        graphs = []
        side = torch.cuda.Stream(dev)  # the legacy default stream cannot be captured
        for j, op in enumerate(oplist):
            row = []
            for s_i in range(nsets):
                ops.reset_launch_count()
                row.append(RawGraph(torch, side, lambda: op.run(dsets[s_i])))
                if s_i == 0:
                    launches_per_step += ops.launch_count()
            graphs.append(row)
        # one graph per buffer set holding the whole step (all operators back to back): the timed region replays
        # these, so the GPU is not idle between operators while the host launches the next graph
        # Operators that share no output buffer (and no workspace) go on parallel branches of the graph: the tail of
        # one kernel then overlaps the head of the next instead of waiting for it.
        outs = [set(op.outputs) for op in oplist]
        parallel = (wname in ("cfg2", "cfg3", "cfg5", "adj2", "adj3", "adj4", "adj5") and not args.serial_step and
                    all(outs[a].isdisjoint(outs[b]) for a in range(len(outs)) for b in range(a)))
        branches = [torch.cuda.Stream(dev) for _ in oplist] if parallel else []

        def step_fn(s_i):
            if not parallel:
                for op in oplist:
                    op.run(dsets[s_i])
                return
            keep = []  # events stay alive until the capture ends
            fork = torch.cuda.Event()
            fork.record(side)
            keep.append(fork)
            for op, st in zip(oplist, branches):
                st.wait_event(fork)
                with torch.cuda.stream(st):
                    op.run(dsets[s_i])
                join = torch.cuda.Event()
                join.record(st)
                side.wait_event(join)
                keep.append(join)
            return keep
        step_graphs = [RawGraph(torch, side, lambda: step_fn(s_i)) for s_i in range(nsets)]
        torch.cuda.synchronize(dev)
        run_op = lambda j, s_i: graphs[j][s_i].replay(stream)  # noqa: E731
    else:
        run_op = lambda j, s_i: oplist[j].run(dsets[s_i])  # noqa: E731
    for i in range(args.warmup):
        for j in range(len(oplist)):
            run_op(j, i % nsets)
    barrier()
    # ---- per-operator breakdown --------------------------------------------------------------------------------
    # An operator's time is the average over back-to-back launches on all buffer sets between one pair of events
    # (the sets rotate, so every launch still reads its inputs from HBM); bracketing single ~50 us launches would
    # add the few microseconds it takes the host to get the next graph launch to an idle GPU.
    bsteps = max(1, min(steps, 50) // nsets)
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in oplist]
          for _ in range(bsteps)]
    for i in range(bsteps):
        for j in range(len(oplist)):
            ev[i][j][0].record(stream)
            for s_i in range(nsets):
                run_op(j, s_i)
            ev[i][j][1].record(stream)
    barrier()
    per_op_ms = [statistics.mean(ev[i][j][0].elapsed_time(ev[i][j][1]) for i in range(bsteps)) / nsets
                 for j in range(len(oplist))]
    # ---- the timed region: exactly args.steps steps ---------------------------------------------------------
    if step_graphs is not None:
        for i in range(args.warmup):
            step_graphs[i % nsets].replay(stream)
    barrier()
    sampler = ClockSampler(dev.index if dev.index is not None else 0)
    sampler.start()
    ops.reset_launch_count()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record(stream)
    for i in range(steps):
        s_i = (args.warmup + i) % nsets
        if step_graphs is not None:
            step_graphs[s_i].replay(stream)
        else:
            for j in range(len(oplist)):
                run_op(j, s_i)
    t_end.record(stream)
    barrier()
    launches = launches_per_step * steps if use_graph else ops.launch_count()
    clocks = sampler.stop()
    total_ms = t_start.elapsed_time(t_end)
    from opscv_b200 import sharding  # the box time of a step is that of its slowest rank
    reduced = sharding.max_over_ranks([total_ms] + per_op_ms, dist, dev)
    total_ms, per_op_ms = reduced[0], reduced[1:]
    step_ms = total_ms / steps
    step_bytes = sum(op.algo_bytes for op in oplist)
    step_pix = sum(op.pixels for op in oplist)
    op_rows = {}
    for op, ms in zip(oplist, per_op_ms):
        gbs = op.algo_bytes / (ms * 1e-3) / 1e9
        op_rows[op.name] = {"ms": ms, "gb_per_s": gbs, "frac_of_peak": gbs / peak, "mpix_per_s": op.pixels / ms / 1e3,
                            "algorithmic_bytes": op.algo_bytes}
        if shard is None and args.batch_div == 1 and NCU_TRAFFIC.get((wname, op.name)) is not None:
            op_rows[op.name]["traffic_from_profile"] = NCU_TRAFFIC[(wname, op.name)]
            op_rows[op.name]["traffic_source"] = TRAFFIC_SOURCE_OP.get((wname, op.name), TRAFFIC_SOURCE.get(wname[:4]))
    dom = max(zip(oplist, per_op_ms), key=lambda p: p[1])
    dom_row = op_rows[dom[0].name]
    roofline = {"kernel": dom[0].name, "bound": "hbm", "achieved": dom_row["gb_per_s"], "peak": peak, "unit": "GB/s",
                "frac": dom_row["frac_of_peak"], "traffic": dom_row.get("traffic_from_profile"),
                "traffic_source": (dom_row.get("traffic_source", "") + " (ncu capture of this kernel; a constant from "
                                   "that capture, not measured in this run)") if "traffic_source" in dom_row else None,
                "share_of_step": dom[1] / sum(per_op_ms)}
    if use_graph:
        del graphs, step_graphs

    # ---- end-to-end arm: host buffers, copies inside the timed region ----------------------------------------
    e2e = None
    if do_e2e:
        pinned = {k: v.pin_memory() for k, v in host.items()}
        in_names = sorted({n for op in oplist for n in op.inputs})
        out_names = sorted({n for op in oplist for n in op.outputs})
        h2d = sum(nbytes(host[n]) for n in in_names)
        d2h = sum(nbytes(host[n]) for n in out_names)
        e2e_steps = max(3, min(steps, 10))

        # Copies and kernels are pipelined the way a caller of an asynchronous API would: host->device copies on one
        # stream, the operators on the compute stream, device->host copies on a third, chained by events, so that
        # the two PCIe directions and the kernels overlap. Every step still moves all its inputs in and all its
        # outputs out inside the timed region.
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        set_free = {}  # buffer set id -> event after which the set may be overwritten again

        def e2e_step(bufs):
            free = set_free.get(id(bufs))
            if free is not None:
                s_in.wait_event(free)
                stream.wait_event(free)
            copied = set()
            last_out = None
            reading = {}  # output buffer -> event of the device->host copy that still reads it
            for op in oplist:
                for n in op.outputs:
                    if n in reading:
                        stream.wait_event(reading[n])
                todo = [n for n in op.inputs if n not in copied]
                if todo:
                    with torch.cuda.stream(s_in):
                        for n in todo:
                            bufs[n].copy_(pinned[n], non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record(s_in)
                    copied.update(todo)
                    stream.wait_event(ev)
                op.run(bufs)
                done = torch.cuda.Event()
                done.record(stream)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(done)
                    for n in op.outputs:
                        pinned[n].copy_(bufs[n], non_blocking=True)
                    last_out = torch.cuda.Event()
                    last_out.record(s_out)
                for n in op.outputs:
                    reading[n] = last_out
            set_free[id(bufs)] = last_out
            return last_out
        for i in range(3):
            e2e_step(dsets[i % nsets])
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for i in range(e2e_steps):
            last = e2e_step(dsets[i % nsets])
        stream.wait_event(last)  # the last outputs have reached the host
        b.record(stream)
        barrier()
        ms = a.elapsed_time(b)
        ms = sharding.max_over_ranks([ms], dist, dev)[0]
        e2e = {"value": world * step_bytes * e2e_steps / (ms * 1e-3) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms / e2e_steps,
               "steps": e2e_steps}
    del dsets
    return {"value": world * step_bytes / (step_ms * 1e-3) / 1e9, "ms_per_step": step_ms,
            "mpix_per_s": world * step_pix / step_ms / 1e3, "ops": op_rows, "roofline": roofline, "e2e": e2e,
            "gpu_launches": int(launches), "clocks": clocks, "config": cfg, "l2_note": note, "steps": steps}


if __name__ == "__main__":
    main()
