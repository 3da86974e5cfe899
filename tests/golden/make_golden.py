#!/usr/bin/env python3
"""Regenerates the golden fixtures in this folder.  Needs the reference tree.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py [--reference /path/to/reference]

What it pins, and against what:

* ``msda_small.npz``    small MSDA cases; expected outputs come from the REAL
  reference evaluator ``gac.core.ops.evaluate_op`` imported from the reference
  tree.  While writing them the script asserts that both restatements under
  ``oracle/`` (NumPy and C) are bit-identical to the reference.  Cases: the
  reference's own known-answer tests (tests/test_bevformer_msda.py:173-264),
  the native fixture recipes (native/tests/generate_base_ops_models.py:200-235),
  the tiny-profile seed-3070 slice shape (tests/test_cuda_gpu.py:39-58, cut
  down), and cut-down versions of the five benchmark configurations.
* ``msda_offsets.npz``  fused-coordinate cases after the recipes of
  native/tests/generate_msda_offsets_models.py:24-141; expected outputs come
  from torch ``grid_sample`` (the independent reference those recipes use) and
  are cross-checked against the reference evaluator fed materialised locations.
* ``msda_softmax.npz``  MSDA with the preceding Softmax node folded in: expected
  outputs are the reference's ``Softmax`` op followed by its
  ``MSDeformableAttention`` op (``--only softmax`` rewrites just this file).
* ``msda_reduce.npz``   MSDA followed by the reference's Mul/ReduceSum/Clamp/Div
  (camera average) or ReduceMean (queue mean) ops (``--only reduce``).
* ``msda_full_pins.npz`` for the four full-size MSDA configurations: 4096
  seeded output positions with the reference evaluator's values plus a float64
  checksum, so a GPU box without the reference tree can still pin full size.
* ``dcn_small.npz``     DCNv2 recipes of generate_base_ops_models.py:85-138 and
  generate_cuda_convolution_models.py:98-130; expected outputs come from
  ``torchvision.ops.deform_conv2d`` (CPU), the operator the reference pins its
  DCNv2 fixtures against; the C oracle is asserted within rtol=atol=2e-5.
* ``dcn_fused.npz``     DCNv2 with Sigmoid (mask), BatchNorm and ReLU folded in:
  expected = the reference's ``Sigmoid`` op, torchvision's operator, then the
  reference's ``BatchNorm`` and ``ReLU`` ops (``--only dcn_fused``).
* ``conv_small.npz``    plain Conv2D cases (grouped/strided/dilated with four pads, a 27-channel
  ``conv_offset`` shape, Conv2D -> ReLU): expected outputs come from the reference's own
  NumPy ``Conv2D`` (and ``ReLU``) evaluator, cross-checked against torch conv2d; the C
  oracle is asserted within 1e-5 (``--only conv``).
* ``dcn_full_pins.npz`` 4096 output positions of the two full-size DCNv2
  configurations from torchvision's CPU operator.
"""

from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("GAC_REFERENCE"), required="GAC_REFERENCE" not in os.environ,
                    help="checkout of the reference project (its src/ must be importable); default: $GAC_REFERENCE")
    ap.add_argument("--only", default="", help="write just one fixture file: 'softmax', 'dcn_fused', 'reduce' or 'conv'")
    args = ap.parse_args()
    sys.dont_write_bytecode = True
    sys.path.insert(0, str(Path(args.reference) / "src"))

    import torch
    import torch.nn.functional as F
    import torchvision

    from gac.core.ops import evaluate_op as ref_evaluate_op  # the real reference

    from general_ai_compiler_b200.bevformer import (WORKLOADS, MsdaWorkload, build_msda_graph,
                                                    make_msda_inputs, make_workload_inputs)
    from oracle import conv2d_c, dcnv2_c, msda_c
    from oracle.msda_numpy import (msda_forward, msda_logits_forward, msda_offsets_forward, sca_camera_average,
                                   tsa_queue_mean)

    torch.set_num_threads(8)

    def ref_msda(value, loc, attn, shapes):
        (out,) = ref_evaluate_op("MSDeformableAttention", (value, loc, attn),
                                 {"spatial_shapes": [list(s) for s in shapes]})
        return out

    def grid_sample_msda(value, shapes, loc, attn):
        """MSDA via torch grid_sample (bilinear, zeros, align_corners=False)."""
        value, loc, attn = map(torch.from_numpy, (value, loc, attn))
        b, _, h, d = value.shape
        q, p = loc.shape[1], loc.shape[4]
        cols, start = [], 0
        for lvl, (hh, ww) in enumerate(shapes):
            feat = value[:, start:start + hh * ww].permute(0, 2, 3, 1).reshape(b * h, d, hh, ww)
            grid = loc[:, :, :, lvl].permute(0, 2, 1, 3, 4).reshape(b * h, q, p, 2) * 2 - 1
            cols.append(F.grid_sample(feat, grid, mode="bilinear", padding_mode="zeros", align_corners=False))
            start += hh * ww
        w = attn.permute(0, 2, 1, 3, 4).reshape(b * h, 1, q, len(shapes) * p)
        out = (torch.stack(cols, dim=-2).flatten(-2) * w).sum(-1)
        return out.reshape(b, h * d, q).transpose(1, 2).contiguous().numpy()

    # ------------------------------------------------------------------ plain Conv2D (the convolutions beside DCNv2)
    # expected = the reference's NumPy Conv2D evaluator (src/gac/core/ops.py:1045-1076), plus its ReLU op for the
    # conv2d_relu case; torch conv2d is an independent cross-check.
    if args.only in ("", "conv"):
        cv = {}
        r = np.random.default_rng(2718)
        cases = (
            # name, X shape, W shape, strides, pads(t,l,b,r), dilations, groups, bias, relu
            ("grouped_strided_dilated", (2, 6, 7, 9), (8, 3, 3, 3), (2, 1), (1, 2, 0, 1), (1, 2), 2, True, False),
            ("pointwise_no_bias", (1, 5, 4, 6), (7, 5, 1, 1), (1, 1), (0, 0, 0, 0), (1, 1), 1, False, False),
            ("conv_offset_small", (1, 16, 9, 11), (27, 16, 3, 3), (1, 1), (1, 1, 1, 1), (1, 1), 1, True, False),
            ("conv_offset_tensor_path", (1, 64, 24, 30), (27, 64, 3, 3), (1, 1), (1, 1, 1, 1), (1, 1), 1, True, False),
            ("conv_relu_tensor_path", (1, 64, 20, 26), (48, 64, 3, 3), (1, 1), (1, 1, 1, 1), (1, 1), 1, True, True),
        )
        for name, xs, ws, st, pads, dil, groups, use_bias, relu in cases:
            x = r.standard_normal(xs).astype(np.float32)
            w = (r.standard_normal(ws) * np.sqrt(2.0 / (ws[1] * ws[2] * ws[3]))).astype(np.float32)
            b = r.standard_normal(ws[0]).astype(np.float32) if use_bias else None
            attrs = {"strides": list(st), "pads": list(pads), "dilations": list(dil), "groups": groups}
            (y,) = ref_evaluate_op("Conv2D", (x, w, b) if use_bias else (x, w), attrs)
            if relu:
                (y,) = ref_evaluate_op("ReLU", (y,), {})
            with torch.inference_mode():
                xt = F.pad(torch.from_numpy(x), (pads[1], pads[3], pads[0], pads[2]))
                yt = F.conv2d(xt, torch.from_numpy(w), None if b is None else torch.from_numpy(b), stride=st,
                              dilation=dil, groups=groups)
                yt = (F.relu(yt) if relu else yt).numpy()
            np.testing.assert_allclose(y, yt, rtol=2e-5, atol=2e-5)
            mine = conv2d_c(x, w, b, strides=st, pads=pads, dilations=dil, groups=groups, relu=relu)
            np.testing.assert_allclose(mine, y, rtol=1e-5, atol=1e-5)
            cv[f"{name}/X"], cv[f"{name}/W"], cv[f"{name}/expected"] = x, w, y.astype(np.float32)
            if use_bias:
                cv[f"{name}/bias"] = b
            cv[f"{name}/attrs"] = np.asarray([*st, *pads, *dil, groups, int(relu)], np.int32)
            print(f"conv {name}: out {y.shape}, max|oracle-ref| {np.abs(mine - y).max():.2e}")
        np.savez_compressed(HERE / "conv_small.npz", **cv)
        if args.only == "conv":
            return

    # ------------------------------------------------------------------ MSDA + the reductions that follow it
    # expected = the reference's MSDeformableAttention, then its Mul/ReduceSum/Clamp/Div (spatial.py:183-188) or
    # ReduceMean (temporal.py:374-389) ops.
    if args.only in ("", "reduce"):
        rd = {}
        r = np.random.default_rng(777)
        b, cams, q, hh, d, p = 2, 3, 24, 8, 32, 4
        sp = [(6, 10), (3, 5)]
        s_total = sum(x * y for x, y in sp)
        value = r.standard_normal((b * cams, s_total, hh, d)).astype(np.float32)
        loc = r.uniform(-0.1, 1.1, (b * cams, q, hh, len(sp), p, 2)).astype(np.float32)
        attn = r.uniform(0, 1, (b * cams, q, hh, len(sp), p)).astype(np.float32)
        attn /= attn.sum(axis=(-1, -2), keepdims=True)
        vis = (r.uniform(0, 1, (b, cams, q, 1)) < 0.3).astype(np.float32)
        vis[0, :, 0] = 0          # a query no camera sees: count clamps to 1, result 0
        vis[1, :, 1] = 1          # a query every camera sees
        vis[0, :, 2, 0] = [1, 0, 1]
        ctx = ref_msda(value, loc, attn, sp)
        (masked,) = ref_evaluate_op("Mul", (ctx.reshape(b, cams, q, hh * d), vis), {})
        (total,) = ref_evaluate_op("ReduceSum", (masked,), {"axes": [1], "keepdims": False})
        (count,) = ref_evaluate_op("ReduceSum", (vis,), {"axes": [1], "keepdims": False})
        (safe,) = ref_evaluate_op("Clamp", (count,), {"min": 1.0})
        (avg,) = ref_evaluate_op("Div", (total, safe), {})
        assert np.array_equal(sca_camera_average(ctx, vis, cams), avg)
        for k, v in (("value", value), ("loc", loc), ("attn", attn), ("visibility", vis), ("expected", avg),
                     ("shapes", np.asarray(sp, np.int32)), ("group", np.asarray(cams, np.int32))):
            rd[f"sca/{k}"] = v
        b, queue, q, p = 1, 2, 49, 4
        sp = [(7, 7)]
        value = r.standard_normal((b * queue, 49, hh, d)).astype(np.float32)
        loc = r.uniform(-0.1, 1.1, (b * queue, q, hh, 1, p, 2)).astype(np.float32)
        attn = r.uniform(0, 1, (b * queue, q, hh, 1, p)).astype(np.float32)
        attn /= attn.sum(axis=(-1, -2), keepdims=True)
        ctx = ref_msda(value, loc, attn, sp)
        (mean,) = ref_evaluate_op("ReduceMean", (ctx.reshape(b, queue, q, hh * d),), {"axes": [1], "keepdims": False})
        assert np.array_equal(tsa_queue_mean(ctx, queue), mean)
        for k, v in (("value", value), ("loc", loc), ("attn", attn), ("expected", mean),
                     ("shapes", np.asarray(sp, np.int32)), ("group", np.asarray(queue, np.int32))):
            rd[f"tsa/{k}"] = v
        np.savez_compressed(HERE / "msda_reduce.npz", **rd)
        if args.only == "reduce":
            return

    # ------------------------------------------------------------------ DCNv2 with Sigmoid / BatchNorm / ReLU folded in
    # expected = the reference's Sigmoid op -> torchvision deform_conv2d (the reference's golden source for DCNv2)
    # -> the reference's BatchNorm op -> the reference's ReLU op.
    if args.only in ("", "dcn_fused"):
        from general_ai_compiler_b200.bevformer import DcnWorkload
        fz = {}
        for name, wl, use_bn, use_relu in (("small_direct", DcnWorkload("f1", 2, 8, 7, 9, 12, seed=901), True, True),
                                           ("tensor_path", DcnWorkload("f2", 1, 64, 24, 30, 96, seed=902), True, True),
                                           ("sigmoid_only", DcnWorkload("f3", 1, 64, 24, 30, 64, seed=903), False, False)):
            x = make_workload_inputs(wl)
            r = np.random.default_rng(wl.seed)
            logits = r.standard_normal(x["mask"].shape).astype(np.float32) * 2
            (mask,) = ref_evaluate_op("Sigmoid", (logits,), {})
            with torch.inference_mode():
                y = torchvision.ops.deform_conv2d(torch.from_numpy(x["X"]), torch.from_numpy(x["offset"]),
                                                  torch.from_numpy(x["W"]), torch.from_numpy(x["bias"]), stride=wl.stride,
                                                  padding=wl.padding, dilation=wl.dilation, mask=torch.from_numpy(mask)).numpy()
            bn = [r.uniform(0.5, 1.5, wl.cout).astype(np.float32), r.standard_normal(wl.cout).astype(np.float32),
                  r.standard_normal(wl.cout).astype(np.float32) * 0.2, r.uniform(0.3, 2.0, wl.cout).astype(np.float32)]
            if use_bn:
                (y,) = ref_evaluate_op("BatchNorm", (y, *bn), {"epsilon": 1e-5})
            if use_relu:
                (y,) = ref_evaluate_op("ReLU", (y,), {})
            for k, v in (("X", x["X"]), ("offset", x["offset"]), ("mask_logits", logits), ("W", x["W"]), ("bias", x["bias"]),
                         ("bn_scale", bn[0]), ("bn_bias", bn[1]), ("bn_mean", bn[2]), ("bn_var", bn[3]),
                         ("flags", np.asarray([int(use_bn), int(use_relu)], np.int32)), ("expected", y)):
                fz[f"{name}/{k}"] = v
        np.savez_compressed(HERE / "dcn_fused.npz", **fz)
        if args.only == "dcn_fused":
            return

    # ------------------------------------------------------------------ MSDA with the Softmax node folded in
    # expected = the reference's Softmax op followed by its MSDeformableAttention op, as in
    # src/gac/models/bevformer/spatial.py:172-182 (scores reshaped to [..., L*P], Softmax(axis=-1), reshaped back).
    sm = {}
    r = np.random.default_rng(4242)
    for name, (b, hh, d, q, p, sp, scale) in {
        "sca_like": (2, 8, 32, 20, 8, [(12, 20), (6, 10), (3, 5), (2, 3)], 1.0),
        "tsa_like": (2, 8, 32, 36, 4, [(9, 9)], 1.0),
        "large_scores": (1, 2, 8, 7, 5, [(4, 3), (2, 2)], 30.0),       # max-subtraction matters
        "odd_dim": (1, 3, 6, 5, 3, [(3, 4)], 2.0),
    }.items():
        s_total = sum(x * y for x, y in sp)
        value = r.standard_normal((b, s_total, hh, d)).astype(np.float32)
        loc = r.uniform(-0.1, 1.1, (b, q, hh, len(sp), p, 2)).astype(np.float32)
        logits = (r.standard_normal((b, q, hh, len(sp), p)) * scale).astype(np.float32)
        (prob,) = ref_evaluate_op("Softmax", (logits.reshape(b, q, hh, len(sp) * p),), {"axis": -1})
        expected = ref_msda(value, loc, prob.reshape(logits.shape), sp)
        assert np.array_equal(msda_logits_forward(value, loc, logits, sp), expected), name
        for k, v in (("value", value), ("loc", loc), ("logits", logits), ("shapes", np.asarray(sp, np.int32)),
                     ("expected", expected)):
            sm[f"{name}/{k}"] = v
    np.savez_compressed(HERE / "msda_softmax.npz", **sm)
    if args.only == "softmax":
        return

    # ------------------------------------------------------------------ MSDA small
    msda = {}

    def add_msda(name, value, loc, attn, shapes, check_grid=True):
        value, loc, attn = (np.ascontiguousarray(a, np.float32) for a in (value, loc, attn))
        expected = ref_msda(value, loc, attn, shapes)
        assert np.array_equal(msda_forward(value, loc, attn, shapes), expected), name
        assert np.array_equal(msda_c(value, loc, attn, shapes), expected), name
        if check_grid:
            np.testing.assert_allclose(grid_sample_msda(value, shapes, loc, attn), expected, rtol=2e-5, atol=2e-5)
        msda[f"{name}/value"] = value
        msda[f"{name}/loc"] = loc
        msda[f"{name}/attn"] = attn
        msda[f"{name}/shapes"] = np.asarray(shapes, np.int32)
        msda[f"{name}/expected"] = expected

    # reference KATs (tests/test_bevformer_msda.py:173-264), restated as data
    add_msda("kat_center_1x1", np.asarray([[[[7.25, -3.5]]]]), np.full((1, 1, 1, 1, 1, 2), 0.5),
             np.ones((1, 1, 1, 1, 1)), [(1, 1)])
    assert np.array_equal(msda["kat_center_1x1/expected"], np.asarray([[[7.25, -3.5]]], np.float32))
    add_msda("kat_2x2_bilinear_padding", np.asarray([1.0, 2.0, 3.0, 4.0]).reshape(1, 4, 1, 1),
             np.asarray([[0.25, 0.25], [0.5, 0.5], [0.0, 0.0], [1.5, 1.5]]).reshape(1, 4, 1, 1, 1, 2),
             np.ones((1, 4, 1, 1, 1)), [(2, 2)])
    np.testing.assert_allclose(msda["kat_2x2_bilinear_padding/expected"][..., 0], [[1.0, 2.5, 0.25, 0.0]], atol=1e-7)
    loc_ml = np.asarray([[
        [[[[0.25, 0.5], [0.75, 0.5]], [[0.5, 0.25], [0.5, 0.75]]],
         [[[0.0, 0.5], [1.0, 0.5]], [[0.5, 0.0], [0.5, 1.0]]]],
        [[[[0.5, 0.5], [1.25, 0.5]], [[0.5, 0.5], [0.5, 1.25]]],
         [[[0.25, 0.5], [0.75, 0.5]], [[0.5, 0.25], [0.5, 0.75]]]],
    ]])
    attn_ml = np.asarray([[
        [[[0.10, 0.20], [0.30, 0.40]], [[0.40, 0.30], [0.20, 0.10]]],
        [[[0.25, 0.25], [0.25, 0.25]], [[0.05, 0.15], [0.35, 0.45]]],
    ]])
    add_msda("kat_multilevel_heads", np.arange(1, 17, dtype=np.float32).reshape(1, 4, 2, 2), loc_ml, attn_ml,
             [(1, 2), (2, 1)])

    rng = np.random.default_rng(20261016)

    def native_recipe(name, *, batch, heads, channels, queries, points, spatial, known_pixels=False):
        spatial = [tuple(s) for s in spatial]
        levels = len(spatial)
        elements = sum(h * w for h, w in spatial)
        value = (rng.standard_normal((batch, elements, heads, channels)) * 0.5).astype(np.float32)
        loc = rng.uniform(-0.25, 1.25, (batch, queries, heads, levels, points, 2)).astype(np.float32)
        attn = rng.uniform(0.1, 1, (batch, queries, heads, levels, points)).astype(np.float32)
        attn /= attn.sum(axis=(-1, -2), keepdims=True)
        loc.reshape(-1, 2)[:4] = [[0, 0], [1, 1], [-1, 0.5], [2, 0.5]]   # exact borders, fully outside
        attn[0, -1] = 0                                                  # a query with zero weights
        if known_pixels:
            loc[0, :, 0, 0, 0] = [[0.25, 0.25], [0.75, 0.25], [0.25, 0.75], [0.75, 0.75]]
            attn.fill(1)
        add_msda(name, value, loc, attn, spatial)
        if known_pixels:
            assert np.array_equal(msda[f"{name}/expected"], value.reshape(1, 4, channels))

    native_recipe("native_exact_pixel_centers", batch=1, heads=1, channels=4, queries=4, points=1,
                  spatial=[(2, 2)], known_pixels=True)
    native_recipe("native_multilevel_heads", batch=1, heads=2, channels=3, queries=3, points=2,
                  spatial=[(2, 3), (1, 2)])
    native_recipe("native_batch_three_levels", batch=2, heads=3, channels=2, queries=4, points=3,
                  spatial=[(3, 2), (1, 4), (2, 1)])
    # the Vortex interpreter case (tests/test_vortex_spatial_ops.py:118-123): 2 levels, U(-0.4, 1.4)
    r13 = np.random.default_rng(13)
    add_msda("two_levels_wide_uniform", r13.standard_normal((2, 8, 2, 4)),
             r13.uniform(-0.4, 1.4, (2, 5, 2, 2, 3, 2)),
             r13.uniform(0.1, 1.0, (2, 5, 2, 2, 3)), [(2, 3), (1, 2)])

    # cut-down benchmark configurations (same level pyramids / distributions, fewer queries)
    for key, q in (("tiny_tsa", 48), ("tiny_sca", 40), ("base_sca", 24), ("base_tsa", 64)):
        w = WORKLOADS[key]
        small = MsdaWorkload(w.name, 2, q, w.heads, w.head_dim, w.points, w.spatial_shapes, w.location_model,
                             w.sigma, w.seed + 1000)
        if key == "base_sca":   # keep the 4-level pyramid but shrink it
            small = MsdaWorkload(w.name, 2, q, 8, 32, 8, ((12, 20), (6, 10), (3, 5), (2, 3)), w.location_model,
                                 0.05, w.seed + 1000)
        if key == "base_tsa":
            small = MsdaWorkload(w.name, 2, q, 8, 32, 4, ((8, 8),), "bev_grid", 0.06, w.seed + 1000)
        if key == "tiny_tsa":
            small = MsdaWorkload(w.name, 2, q, 8, 32, 4, ((10, 10),), "uniform", 0.0, w.seed + 1000)
        x = make_workload_inputs(small)
        add_msda(f"cfg_{key}", x["value"], x["sampling_locations"], x["attention_weights"], small.spatial_shapes)
    # odd extents: H=3 heads, D=5, D=12 (vector path with 3 lanes is not a power of two), P=3, many points
    r = np.random.default_rng(987)
    for name, (b, hh, d, q, p, sp) in {
        "odd_heads_dim5": (1, 3, 5, 7, 3, [(4, 3), (2, 2)]),
        "dim12": (2, 2, 12, 9, 2, [(5, 4)]),
        "dim64_points40": (1, 2, 64, 5, 40, [(6, 7)]),
        "dim8_one_point": (3, 4, 8, 33, 1, [(3, 3), (2, 2)]),
        "dim128": (1, 1, 128, 6, 4, [(4, 4)]),
    }.items():
        s = sum(a * c for a, c in sp)
        add_msda(name, r.standard_normal((b, s, hh, d)), r.uniform(-0.3, 1.3, (b, q, hh, len(sp), p, 2)),
                 r.uniform(0, 1, (b, q, hh, len(sp), p)), sp)
    # tiny-profile slice recipe (seed 3070), first 16 queries of 2 cameras
    g = build_msda_graph()
    full = make_msda_inputs(g, seed=3070)
    add_msda("tiny_profile_seed3070_cut", full["value"][:2], full["sampling_locations"][:2, :16],
             full["attention_weights"][:2, :16], [(15, 25)])
    np.savez_compressed(HERE / "msda_small.npz", **msda)

    # ------------------------------------------------------------------ MSDA fused coordinates
    off = {}
    rng = np.random.default_rng(50841)
    batch, queries, heads, levels, points, channels = 2, 3, 2, 2, 4, 3
    loc_shape = (batch, queries, heads, levels, points, 2)
    shapes = [(2, 3), (1, 2)]

    def offsets_case(name, *, spatial=False, first=False, full_norm=False, special_norm=False):
        coord_shape = (batch, queries, heads, levels, points // 2, 2, 2) if spatial else loc_shape
        ref_shape = (batch, queries, 1, 1, 1, 2, 2) if spatial else (batch, queries, 1, 1, 1, 2)
        value = rng.uniform(-1, 1, (batch, 8, heads, channels)).astype(np.float32)
        offsets = rng.uniform(-1.5, 1.5, loc_shape).astype(np.float32)
        normalizer = np.array([3, 2, 2, 1], np.float32).reshape(1, 1, 1, levels, 1, 2)
        reference = rng.uniform(0.1, 0.9, ref_shape).astype(np.float32)
        weights = rng.uniform(0.05, 1, (batch, queries, heads, levels, points)).astype(np.float32)
        weights /= weights.sum(axis=(-1, -2), keepdims=True)
        weights[0, -1] = 0
        if full_norm:
            normalizer = rng.uniform(0.25, 4, loc_shape).astype(np.float32)
            normalizer[..., 1] *= -1
        if special_norm:
            normalizer = np.broadcast_to(normalizer, loc_shape).copy()
            normalizer[0, 0, 0, :, 0, :] = [[np.inf, -np.inf], [0.125, -0.25]]
        with torch.inference_mode():
            t_div = torch.from_numpy(offsets) / torch.from_numpy(normalizer)
            t_view = t_div.reshape(coord_shape)
            t_ref = torch.from_numpy(reference)
            t_loc = ((t_ref + t_view) if first else (t_view + t_ref)).reshape(loc_shape).contiguous().numpy()
        expected = grid_sample_msda(value, shapes, t_loc, weights)
        via_ref = ref_msda(value, t_loc, weights, shapes)
        np.testing.assert_allclose(via_ref, expected, rtol=2e-5, atol=2e-5)
        port = msda_offsets_forward(value, offsets, weights, normalizer, reference, shapes, coord_shape, first)
        assert np.array_equal(port, via_ref), name
        for k, v in (("value", value), ("offsets", offsets), ("normalizer", normalizer), ("reference", reference),
                     ("weights", weights), ("expected", via_ref), ("expected_grid_sample", expected),
                     ("shapes", np.asarray(shapes, np.int32)), ("coordinate_shape", np.asarray(coord_shape, np.int32)),
                     ("reference_first", np.asarray(int(first), np.int32))):
            off[f"{name}/{k}"] = np.ascontiguousarray(v)

    offsets_case("temporal_reference_right")
    offsets_case("temporal_reference_left", first=True)
    offsets_case("spatial_rank_seven_right", spatial=True)
    offsets_case("spatial_rank_seven_left", spatial=True, first=True)
    offsets_case("temporal_full_shape_normalizer", full_norm=True)
    offsets_case("temporal_signed_and_infinite_normalizer", special_norm=True)
    np.savez_compressed(HERE / "msda_offsets.npz", **off)

    # ------------------------------------------------------------------ MSDA full-size pins
    pins = {}
    for key in ("tiny_tsa", "tiny_sca", "base_sca", "base_tsa"):
        w = WORKLOADS[key]
        x = make_workload_inputs(w)
        expected = ref_msda(x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes)
        c_out = msda_c(x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes)
        assert np.array_equal(c_out, expected), key
        idx = np.random.default_rng(w.seed + 7).choice(expected.size, 4096, replace=False).astype(np.int64)
        pins[f"{key}/index"] = idx
        pins[f"{key}/expected"] = expected.reshape(-1)[idx]
        pins[f"{key}/sum64"] = np.asarray(expected.astype(np.float64).sum())
        pins[f"{key}/abs_sum64"] = np.asarray(np.abs(expected.astype(np.float64)).sum())
        print(key, "pinned", expected.shape, float(pins[f"{key}/sum64"]))
    np.savez_compressed(HERE / "msda_full_pins.npz", **pins)

    # ------------------------------------------------------------------ DCNv2 small
    dcn = {}

    def tv_dcn(x, offset, mask, weight, bias, stride, padding, dilation):
        with torch.inference_mode():
            return torchvision.ops.deform_conv2d(
                torch.from_numpy(x), torch.from_numpy(offset), torch.from_numpy(weight),
                None if bias is None else torch.from_numpy(bias), stride=stride, padding=padding,
                dilation=dilation, mask=torch.from_numpy(mask)).numpy()

    def add_dcn(name, x, offset, mask, weight, bias, stride, padding, dilation, groups, dgroups):
        expected = tv_dcn(x, offset, mask, weight, bias, stride, padding, dilation)
        mine = dcnv2_c(x, offset, mask, weight, bias, stride=stride, padding=padding, dilation=dilation,
                       groups=groups, deform_groups=dgroups)
        np.testing.assert_allclose(mine, expected, rtol=2e-5, atol=2e-5, err_msg=name)
        for k, v in (("X", x), ("offset", offset), ("mask", mask), ("W", weight), ("expected", expected),
                     ("attrs", np.asarray([*stride, *padding, *dilation, groups, dgroups], np.int32))):
            dcn[f"{name}/{k}"] = np.ascontiguousarray(v)
        if bias is not None:
            dcn[f"{name}/bias"] = bias
        return expected

    rng = np.random.default_rng(20261016)

    def rnd(shape, scale=0.5):
        return (rng.standard_normal(shape) * scale).astype(np.float32)

    def base_recipe(name, *, batch=1, cin=2, cout=3, height=5, width=6, kernel=(3, 3), stride=(1, 1),
                    padding=(1, 1), dilation=(1, 1), groups=1, dgroups=1, bias=True, zero_offsets=False,
                    fractional_edges=False):
        kh, kw = kernel
        oh = (height + 2 * padding[0] - dilation[0] * (kh - 1) - 1) // stride[0] + 1
        ow = (width + 2 * padding[1] - dilation[1] * (kw - 1) - 1) // stride[1] + 1
        x = rnd((batch, cin, height, width))
        offset = rng.uniform(-0.8, 0.8, (batch, 2 * dgroups * kh * kw, oh, ow)).astype(np.float32)
        mask = rng.uniform(0.05, 1.0, (batch, dgroups * kh * kw, oh, ow)).astype(np.float32)
        weight = rnd((cout, cin // groups, kh, kw))
        b = rnd((cout,)) if bias else None
        mask[..., 0, 0] = 0
        if zero_offsets:
            offset.fill(0)
            mask.fill(1)
        if fractional_edges:
            offset[0, 0] = np.array([[-0.25, -1.0, 0.5], [0.5, 1.0, -0.3]], np.float32)
            offset[0, 1] = np.array([[-0.4, 0.25, 0.5], [-1.0, 0.5, 0.0]], np.float32)
            mask.fill(0.75)
        expected = add_dcn(name, x, offset, mask, weight, b, stride, padding, dilation, groups, dgroups)
        if zero_offsets:
            plain = F.conv2d(torch.from_numpy(x), torch.from_numpy(weight), None if b is None else torch.from_numpy(b),
                             stride=stride, padding=padding, dilation=dilation, groups=groups).numpy()
            np.testing.assert_allclose(expected, plain, rtol=2e-5, atol=2e-5)

    # torchvision's operator takes `groups` from the weight shape, as the recipes rely on.
    base_recipe("dcn_mask_bias")
    base_recipe("dcn_batch_grouped", batch=2, cin=4, cout=6, height=6, width=7, kernel=(2, 3), stride=(2, 1),
                padding=(1, 0), dilation=(2, 1), groups=2, dgroups=2)
    base_recipe("dcn_four_deform_groups", cin=4, cout=4, height=7, width=8, kernel=(3, 2), stride=(1, 2),
                padding=(2, 1), dilation=(2, 1), dgroups=4, bias=False)
    base_recipe("dcn_zero_offset_conv_equivalence", cin=4, cout=4, groups=2, dgroups=1, zero_offsets=True, bias=False)
    base_recipe("dcn_fractional_zero_padding", cin=1, cout=1, height=2, width=3, kernel=(1, 1), padding=(0, 0),
                fractional_edges=True)

    rng = np.random.default_rng(20261017)

    def conv_recipe(name, *, cin=4, cout=8, groups=1, dgroups=1, batch=2, height=6, width=7, bias=True, zero=False):
        kernel, stride, padding, dilation = (3, 2), (1, 1), (1, 1), (1, 1)
        oh, ow = height, width + 1
        x = rnd((batch, cin, height, width))
        offset = rng.uniform(-1.25, 1.25, (batch, 12 * dgroups, oh, ow)).astype(np.float32)
        mask = rng.uniform(0, 1, (batch, 6 * dgroups, oh, ow)).astype(np.float32)
        mask[..., 0, 0] = 0
        if zero:
            offset.fill(0)
            mask.fill(1)
        weight = rnd((cout, cin // groups, *kernel))
        b = rnd((cout,)) if bias else None
        add_dcn(name, x, offset, mask, weight, b, stride, padding, dilation, groups, dgroups)

    conv_recipe("dcn_shared_samples")
    conv_recipe("dcn_groups_and_deform_groups", cin=8, cout=16, groups=2, dgroups=4)
    conv_recipe("dcn_grouped_no_bias", cin=4, cout=16, groups=4, dgroups=2, bias=False)
    conv_recipe("dcn_zero_offsets", zero=True)
    conv_recipe("dcn_odd_group_channels", cin=4, cout=6, groups=2, dgroups=2)
    conv_recipe("dcn_representative_channels", cin=32, cout=64, batch=1, height=16, width=16)
    # cut-down stage shapes: 3x3, stride 1, pad 1, offsets ~ N(0,2) px, sigmoid mask
    from general_ai_compiler_b200.bevformer import DcnWorkload
    for name, wl in (("cfg_dcn_c4_cut", DcnWorkload("c4cut", 2, 64, 13, 20, 96, seed=777)),
                     ("cfg_dcn_c5_cut", DcnWorkload("c5cut", 1, 128, 9, 11, 128, seed=778))):
        x = make_workload_inputs(wl)
        add_dcn(name, x["X"], x["offset"], x["mask"], x["W"], x["bias"], wl.stride, wl.padding, wl.dilation, 1, 1)
    np.savez_compressed(HERE / "dcn_small.npz", **dcn)

    # ------------------------------------------------------------------ DCNv2 full-size pins
    pins = {}
    for key in ("dcn_c4", "dcn_c5"):
        wl = WORKLOADS[key]
        x = make_workload_inputs(wl)
        expected = tv_dcn(x["X"], x["offset"], x["mask"], x["W"], x["bias"], wl.stride, wl.padding, wl.dilation)
        mine = dcnv2_c(x["X"], x["offset"], x["mask"], x["W"], x["bias"], stride=wl.stride, padding=wl.padding,
                       dilation=wl.dilation)
        err = float(np.abs(mine - expected).max())
        assert err < 1e-4, (key, err)
        idx = np.random.default_rng(wl.seed + 7).choice(expected.size, 4096, replace=False).astype(np.int64)
        pins[f"{key}/index"] = idx
        pins[f"{key}/expected"] = expected.reshape(-1)[idx]
        pins[f"{key}/oracle_max_abs_vs_torchvision"] = np.asarray(err)
        print(key, "pinned", expected.shape, "C oracle vs torchvision max abs", err)
    np.savez_compressed(HERE / "dcn_full_pins.npz", **pins)
    print("versions: torch", torch.__version__, "torchvision", torchvision.__version__, "numpy", np.__version__)


if __name__ == "__main__":
    main()
