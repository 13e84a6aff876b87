"""Pins the CPU oracle against the committed golden fixtures (tests/golden/resample_golden.npz, produced by
tests/golden/make_golden.py from the reference's own Python golden and the PyTorch-CPU calls its tests make).

Tolerances: the reference's kernel tests accept rtol 1e-4 (fp32 forward) and 1e-2 (gradients) against the same
PyTorch goldens (image/upsample_bilinear2d/tests/ut/op_kernel/upsample_bilinear2d_data/compare_data.py:23-39).
The oracle is held to a tighter bound here: it and PyTorch evaluate the same formulas in fp32 with different
rounding orders, which leaves differences of a few ulp of the largest operand.
"""
import ast
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "resample_golden.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLDEN)


def _close(a, b, rtol=2e-5, atol=5e-6):
    np.testing.assert_allclose(a, b, rtol=rtol, atol=atol)


def _interp_cases(gold, prefix):
    for m in gold["meta.interp"]:
        name, mode, shape, out, align, scales = ast.literal_eval(str(m))
        if name.startswith(prefix):
            yield name, shape, out, align, scales if scales is not None else (0.0, 0.0)


def test_nearest_matches_golden(oracle, gold):
    n = 0
    for name, shape, out, _, scales in _interp_cases(gold, "nearest."):
        y = oracle.nearest2d_fwd(gold[name + ".x"], out, scales)
        assert np.array_equal(y, gold[name + ".y"]), name  # pure copy: exact
        gx = oracle.nearest2d_bwd(gold[name + ".g"], shape[2:], scales)
        _close(gx, gold[name + ".gx"])
        n += 1
    assert n == 4


def test_bilinear_matches_golden(oracle, gold):
    n = 0
    for name, shape, out, align, scales in _interp_cases(gold, "bilinear."):
        _close(oracle.bilinear2d_fwd(gold[name + ".x"], out, align, scales), gold[name + ".y"])
        for definition in ("scatter", "gather"):
            gx = oracle.bilinear2d_bwd(gold[name + ".g"], shape[2:], align, scales, definition=definition)
            _close(gx, gold[name + ".gx"], atol=1e-5)
        n += 1
    assert n == 8


def test_bilinear_reference_example(oracle, gold):
    # fixed input of the reference's example client (align_corners = true, scales 2.0)
    y = oracle.bilinear2d_fwd(gold["example.bilinear.x"], (8, 4), True, (2.0, 2.0))
    _close(y, gold["example.bilinear.y"])


def test_bicubic_aa_matches_golden(oracle, gold):
    n = 0
    for name, shape, out, align, scales in _interp_cases(gold, "bicubic_aa."):
        _close(oracle.bicubic_aa_fwd(gold[name + ".x"], out, align, scales), gold[name + ".y"], atol=1e-5)
        for definition in ("scatter", "gather"):
            gx = oracle.bicubic_aa_bwd(gold[name + ".g"], shape[2:], align, scales, definition=definition)
            _close(gx, gold[name + ".gx"], atol=1e-5)
        n += 1
    assert n == 5


@pytest.mark.parametrize("mode", ["bilinear", "nearest", "bicubic"])
@pytest.mark.parametrize("pad", ["zeros", "border", "reflection"])
@pytest.mark.parametrize("align", [False, True])
def test_grid_sampler_matches_reference_golden(oracle, gold, mode, pad, align):
    mi = ["bilinear", "nearest", "bicubic"].index(mode)
    pi = ["zeros", "border", "reflection"].index(pad)
    name = f"grid.{mode}.{pad}.{'ac' if align else 'hp'}"
    x, grid = gold[name + ".x"], gold[name + ".grid"]
    y = oracle.grid_sampler2d_fwd(x, grid, mi, pi, align)
    if mode == "nearest":
        assert np.array_equal(y, gold[name + ".y"])
    else:
        _close(y, gold[name + ".y"])
    if mode != "bicubic":
        gx, gg = oracle.grid_sampler2d_bwd(gold[name + ".g"], x, grid, mi, pi, align)
        _close(gx, gold[name + ".gx"])
        _close(gg, gold[name + ".ggrid"], rtol=1e-4, atol=1e-5)


def test_grid_sampler_reference_example(oracle, gold):
    x, grid = gold["example.grid.x"], gold["example.grid.grid"]
    _close(oracle.grid_sampler2d_fwd(x, grid), gold["example.grid.y"])
    gx, gg = oracle.grid_sampler2d_bwd(np.ones_like(gold["example.grid.y"]), x, grid)
    _close(gx, gold["example.grid.gx"])
    _close(gg, gold["example.grid.ggrid"], rtol=1e-4, atol=1e-5)


def test_oracle_edge_shapes(oracle):
    rng = np.random.default_rng(7)
    # 1x1 input broadcast, 1-wide / 1-tall tensors, identity size
    x = rng.standard_normal((1, 2, 1, 1)).astype(np.float32)
    y = oracle.bilinear2d_fwd(x, (3, 5))
    assert np.array_equal(y, np.broadcast_to(x, (1, 2, 3, 5)))
    assert np.array_equal(oracle.nearest2d_fwd(x, (3, 5)), np.broadcast_to(x, (1, 2, 3, 5)))
    x = rng.standard_normal((1, 1, 4, 6)).astype(np.float32)
    assert np.array_equal(oracle.bilinear2d_fwd(x, (4, 6)), x)
    assert np.array_equal(oracle.bicubic_aa_fwd(x, (4, 6)), x)
    assert np.array_equal(oracle.nearest2d_bwd(x, (4, 6)), x)
    # gradient of a sum equals column sums of the weights: sum of grad_input == sum of grad_output (partition of 1)
    g = rng.standard_normal((1, 1, 9, 11)).astype(np.float32)
    for fn in (lambda: oracle.bilinear2d_bwd(g, (4, 5)), lambda: oracle.bicubic_aa_bwd(g, (20, 23)),
               lambda: oracle.nearest2d_bwd(g, (4, 5))):
        np.testing.assert_allclose(fn().sum(dtype=np.float64), g.sum(dtype=np.float64), rtol=1e-5, atol=1e-4)


def test_oracle_tables(oracle):
    # exact 2x up-sampling: known source indices and weights
    idx = oracle.nearest_src_index(4, 8)
    assert idx.tolist() == [0, 0, 1, 1, 2, 2, 3, 3]
    s, e = oracle.nearest_bwd_ranges(4, 8)
    assert s.tolist() == [0, 2, 4, 6] and e.tolist() == [2, 4, 6, 8]
    lo, hi, d = oracle.bilinear_table(4, 8, False)
    assert lo.tolist() == [0, 0, 0, 1, 1, 2, 2, 3]
    assert hi.tolist() == [0, 1, 1, 2, 2, 3, 3, 3]
    np.testing.assert_array_equal(d, np.array([0, .25, .75, .25, .75, .25, .75, .25], dtype=np.float32))
    xmin, xsize, w = oracle.bicubic_aa_table(16, 4, False)
    assert xmin.tolist() == [0, 0, 2, 6] and xsize.tolist() == [10, 14, 14, 10]
    np.testing.assert_allclose(w.sum(axis=1), 1.0, rtol=1e-6)
