"""The CPU oracles against the committed golden vectors (and the reference tree when present)."""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import pytest

from conftest import load_cases
from general_ai_compiler_b200.bevformer import WORKLOADS, make_workload_inputs
from oracle import dcnv2_c, dcnv2_fused_c, msda_c
from oracle.msda_numpy import (OracleError, msda_forward, msda_forward_threaded, msda_logits_forward,
                               msda_offsets_forward)

# checkout of the reference project, named by the GAC_REFERENCE environment variable; without it the test that
# compares against the tree itself is skipped (the committed fixtures hold the reference's outputs)
_REFERENCE = os.environ.get("GAC_REFERENCE", "")
REFERENCE_SRC = Path(_REFERENCE) / "src" if _REFERENCE else None


def _shapes(a):
    return [tuple(int(v) for v in row) for row in a]


@pytest.mark.parametrize("case", sorted(load_cases("msda_small.npz")))
def test_msda_oracles_are_bit_identical_to_reference_outputs(case, msda_small):
    c = msda_small[case]
    shapes = _shapes(c["shapes"])
    assert np.array_equal(msda_forward(c["value"], c["loc"], c["attn"], shapes), c["expected"])
    assert np.array_equal(msda_c(c["value"], c["loc"], c["attn"], shapes), c["expected"])


def test_reference_known_answers(msda_small):
    """The literal expectations of the reference's own tests (tests/test_bevformer_msda.py:173-211)."""
    assert np.array_equal(msda_small["kat_center_1x1"]["expected"], np.asarray([[[7.25, -3.5]]], np.float32))
    np.testing.assert_allclose(msda_small["kat_2x2_bilinear_padding"]["expected"][..., 0],
                               np.asarray([[1.0, 2.5, 0.25, 0.0]], np.float32), rtol=0, atol=1e-7)
    c = msda_small["native_exact_pixel_centers"]
    assert np.array_equal(c["expected"], c["value"].reshape(1, 4, 4))


def test_multilevel_matches_scalar_float64_definition(msda_small):
    """Independent scalar definition, like the in-test one of tests/test_bevformer_msda.py:47-105."""
    c = msda_small["kat_multilevel_heads"]
    value, loc, attn, shapes = c["value"], c["loc"], c["attn"], _shapes(c["shapes"])
    B, _, H, D = value.shape
    Q, L, P = loc.shape[1], loc.shape[3], loc.shape[4]
    out = np.zeros((B, Q, H, D))
    start = 0
    for l, (hh, ww) in enumerate(shapes):
        img = value[:, start:start + hh * ww].reshape(B, hh, ww, H, D)
        start += hh * ww
        for b in range(B):
            for q in range(Q):
                for h in range(H):
                    for p in range(P):
                        x = float(loc[b, q, h, l, p, 0]) * ww - 0.5
                        y = float(loc[b, q, h, l, p, 1]) * hh - 0.5
                        x0, y0 = int(np.floor(x)), int(np.floor(y))
                        for xx, yy, cf in ((x0, y0, (x0 + 1 - x) * (y0 + 1 - y)), (x0 + 1, y0, (x - x0) * (y0 + 1 - y)),
                                           (x0, y0 + 1, (x0 + 1 - x) * (y - y0)), (x0 + 1, y0 + 1, (x - x0) * (y - y0))):
                            if 0 <= xx < ww and 0 <= yy < hh:
                                out[b, q, h] += float(attn[b, q, h, l, p]) * cf * img[b, yy, xx, h]
    np.testing.assert_allclose(c["expected"], out.reshape(B, Q, H * D), rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("case", sorted(load_cases("msda_offsets.npz")))
def test_fused_coordinate_oracle(case, msda_offsets):
    c = msda_offsets[case]
    out = msda_offsets_forward(c["value"], c["offsets"], c["weights"], c["normalizer"], c["reference"],
                               _shapes(c["shapes"]), tuple(c["coordinate_shape"]), bool(c["reference_first"]))
    assert np.array_equal(out, c["expected"])
    np.testing.assert_allclose(out, c["expected_grid_sample"], rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("case", sorted(load_cases("msda_softmax.npz")))
def test_softmax_folded_oracle(case, msda_softmax):
    c = msda_softmax[case]
    assert np.array_equal(msda_logits_forward(c["value"], c["loc"], c["logits"], _shapes(c["shapes"])), c["expected"])


def test_group_reduction_oracles(msda_reduce):
    from oracle.msda_numpy import sca_camera_average, tsa_queue_mean

    c = msda_reduce["sca"]
    ctx = msda_c(c["value"], c["loc"], c["attn"], _shapes(c["shapes"]))
    out = sca_camera_average(ctx, c["visibility"], int(c["group"]))
    assert np.array_equal(out, c["expected"])
    assert not out[0, 0].any()                      # the query no camera sees
    c = msda_reduce["tsa"]
    ctx = msda_c(c["value"], c["loc"], c["attn"], _shapes(c["shapes"]))
    assert np.array_equal(tsa_queue_mean(ctx, int(c["group"])), c["expected"])


@pytest.mark.parametrize("key", ["tiny_tsa", "tiny_sca", "base_sca", "base_tsa"])
def test_full_size_pins_with_c_oracle(key, msda_pins):
    w = WORKLOADS[key]
    x = make_workload_inputs(w)
    out = msda_c(x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes)
    pin = msda_pins[key]
    assert np.array_equal(out.reshape(-1)[pin["index"]], pin["expected"])
    assert out.astype(np.float64).sum() == float(pin["sum64"])


def test_threaded_numpy_oracle_equals_serial():
    w = WORKLOADS["tiny_sca"].with_queries(300)
    x = make_workload_inputs(w)
    args = (x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes)
    assert np.array_equal(msda_forward_threaded(*args, threads=5), msda_forward(*args))


def test_oracle_rejects_inconsistent_shapes():
    v = np.zeros((1, 4, 1, 2), np.float32)
    with pytest.raises(OracleError):
        msda_forward(v, np.zeros((1, 1, 1, 1, 1, 2), np.float32), np.zeros((1, 1, 1, 1, 1), np.float32), [(2, 3)])
    with pytest.raises(ValueError):
        msda_c(v, np.zeros((1, 1, 1, 1, 1, 2), np.float32), np.zeros((1, 1, 1, 1, 1), np.float32), [(2, 3)])


def test_empty_query_set():
    v = np.ones((2, 4, 1, 4), np.float32)
    out = msda_c(v, np.zeros((2, 0, 1, 1, 3, 2), np.float32), np.zeros((2, 0, 1, 1, 3), np.float32), [(2, 2)])
    assert out.shape == (2, 0, 4)
    assert msda_forward(v, np.zeros((2, 0, 1, 1, 3, 2), np.float32), np.zeros((2, 0, 1, 1, 3), np.float32),
                        [(2, 2)]).shape == (2, 0, 4)


@pytest.mark.parametrize("case", sorted(load_cases("dcn_small.npz")))
def test_dcn_oracle_against_torchvision_fixtures(case, dcn_small):
    c = dcn_small[case]
    a = [int(v) for v in c["attrs"]]
    out = dcnv2_c(c["X"], c["offset"], c["mask"], c["W"], c.get("bias"), stride=a[0:2], padding=a[2:4],
                  dilation=a[4:6], groups=a[6], deform_groups=a[7])
    np.testing.assert_allclose(out, c["expected"], rtol=2e-5, atol=2e-5)


def test_dcn_fractional_zero_padding_by_hand(dcn_small):
    """1x1 kernel on a 2x3 image, mask 0.75: every output is 0.75*w*bilinear(x at p+offset)+bias."""
    c = dcn_small["dcn_fractional_zero_padding"]
    img = c["X"][0, 0].astype(np.float64)
    w, b = float(c["W"][0, 0, 0, 0]), float(c["bias"][0])
    for oy in range(2):
        for ox in range(3):
            y = oy + float(c["offset"][0, 0, oy, ox])
            x = ox + float(c["offset"][0, 1, oy, ox])
            y0, x0 = int(np.floor(y)), int(np.floor(x))
            acc = 0.0
            for yy, xx, cf in ((y0, x0, (1 - (y - y0)) * (1 - (x - x0))), (y0, x0 + 1, (1 - (y - y0)) * (x - x0)),
                               (y0 + 1, x0, (y - y0) * (1 - (x - x0))), (y0 + 1, x0 + 1, (y - y0) * (x - x0))):
                if 0 <= yy < 2 and 0 <= xx < 3:
                    acc += cf * img[yy, xx]
            assert abs(c["expected"][0, 0, oy, ox] - (0.75 * acc * w + b)) < 2e-6


@pytest.mark.parametrize("key", ["dcn_c5"])
def test_dcn_full_size_pin(key, dcn_pins):
    wl = WORKLOADS[key]
    x = make_workload_inputs(wl)
    out = dcnv2_c(x["X"], x["offset"], x["mask"], x["W"], x["bias"], stride=wl.stride, padding=wl.padding,
                  dilation=wl.dilation)
    pin = dcn_pins[key]
    np.testing.assert_allclose(out.reshape(-1)[pin["index"]], pin["expected"], rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("case", sorted(load_cases("dcn_fused.npz")))
def test_dcn_fused_oracle(case, dcn_fused):
    c = dcn_fused[case]
    use_bn, use_relu = (bool(v) for v in c["flags"])
    bn = (c["bn_scale"], c["bn_bias"], c["bn_mean"], c["bn_var"], 1e-5) if use_bn else None
    out = dcnv2_fused_c(c["X"], c["offset"], c["mask_logits"], c["W"], c["bias"], bn=bn, relu=use_relu,
                        stride=(1, 1), padding=(1, 1), dilation=(1, 1))
    np.testing.assert_allclose(out, c["expected"], rtol=2e-5, atol=2e-5)


def conv_case_attrs(c):
    a = [int(v) for v in c["attrs"]]
    return dict(strides=tuple(a[0:2]), pads=tuple(a[2:6]), dilations=tuple(a[6:8]), groups=a[8], relu=bool(a[9]))


@pytest.mark.parametrize("case", sorted(load_cases("conv_small.npz")))
def test_conv_oracle_against_reference_evaluator_outputs(case, conv_small):
    """The fixtures hold the outputs of the reference's own NumPy Conv2D (double accumulation); the float32
    restatement of the native lowering must agree within float32 rounding."""
    from oracle import conv2d_c

    c = conv_small[case]
    out = conv2d_c(c["X"], c["W"], c.get("bias"), **conv_case_attrs(c))
    assert out.shape == c["expected"].shape
    np.testing.assert_allclose(out, c["expected"], rtol=1e-5, atol=1e-5)


def test_conv_oracle_equals_zero_offset_dcn_oracle():
    """A deformable convolution with zero offsets and a unit mask is the plain convolution, bit for bit."""
    from oracle import conv2d_c

    rng = np.random.default_rng(12)
    x = rng.standard_normal((2, 4, 6, 7)).astype(np.float32)
    w = rng.standard_normal((6, 4, 3, 3)).astype(np.float32)
    b = rng.standard_normal(6).astype(np.float32)
    plain = conv2d_c(x, w, b, pads=(1, 1, 1, 1))
    dcn = dcnv2_c(x, np.zeros((2, 18, 6, 7), np.float32), np.ones((2, 9, 6, 7), np.float32), w, b, padding=(1, 1))
    assert np.array_equal(plain, dcn)
    with pytest.raises(ValueError):
        conv2d_c(x, np.zeros((6, 2, 3, 3), np.float32), None, groups=4)


def test_dcn_oracle_rejects_bad_groups():
    x = np.zeros((1, 4, 3, 3), np.float32)
    with pytest.raises(ValueError):
        dcnv2_c(x, np.zeros((1, 18, 3, 3), np.float32), np.zeros((1, 9, 3, 3), np.float32),
                np.zeros((3, 4, 3, 3), np.float32), None, padding=(1, 1), groups=3)


@pytest.mark.skipif(REFERENCE_SRC is None or not REFERENCE_SRC.exists(), reason="GAC_REFERENCE does not name a reference checkout")
def test_oracle_equals_real_reference_when_mounted():
    sys.dont_write_bytecode = True
    sys.path.insert(0, str(REFERENCE_SRC))
    try:
        from gac.core.ops import evaluate_op as ref_evaluate_op
    finally:
        sys.path.remove(str(REFERENCE_SRC))
    rng = np.random.default_rng(5)
    shapes = [(5, 7), (3, 2)]
    value = rng.standard_normal((2, 41, 3, 8)).astype(np.float32)
    loc = rng.uniform(-0.3, 1.3, (2, 11, 3, 2, 5, 2)).astype(np.float32)
    attn = rng.uniform(0, 1, (2, 11, 3, 2, 5)).astype(np.float32)
    (ref,) = ref_evaluate_op("MSDeformableAttention", (value, loc, attn), {"spatial_shapes": shapes})
    assert np.array_equal(msda_forward(value, loc, attn, shapes), ref)
    assert np.array_equal(msda_c(value, loc, attn, shapes), ref)


def test_restatements_equal_the_reference_modules_under_oracle_ref():
    """Where oracle/_ref holds the reference's own evaluator (placed there by oracle/make_ref.py), the NumPy and
    C restatements must agree with it bit for bit on a seeded ragged case, through evaluate_op and reference_run."""
    import oracle

    if not oracle.reference_available():
        pytest.skip("oracle/_ref is not populated on this box")
    ref = oracle.load_reference()
    rng = np.random.default_rng(11)
    shapes = [(7, 5), (4, 3), (1, 2)]
    size = sum(h * w for h, w in shapes)
    value = rng.standard_normal((3, size, 2, 8)).astype(np.float32)
    loc = rng.uniform(-0.3, 1.3, (3, 13, 2, 3, 5, 2)).astype(np.float32)
    attn = rng.uniform(0, 1, (3, 13, 2, 3, 5)).astype(np.float32)
    want = ref.evaluate_op("MSDeformableAttention", [value, loc, attn], {"spatial_shapes": [list(s) for s in shapes]})[0]
    assert np.array_equal(msda_forward(value, loc, attn, shapes), want)
    assert np.array_equal(msda_c(value, loc, attn, shapes), want)
    graph = oracle.reference_msda_graph(ref, 3, size, 13, 2, 8, 3, 5, shapes)
    got = ref.reference_run(graph, {"value": value, "sampling_locations": loc, "attention_weights": attn})["output"]
    assert np.array_equal(got, want)
