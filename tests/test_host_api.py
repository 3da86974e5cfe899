"""Host-side contract tests: shape inference, graph types, launch planning, input binding.

Written after the reference's contract tests (tests/test_bevformer_msda.py:108-169, :267-336) so
that the same expectations hold for this package's API.  No GPU is needed.
"""

from __future__ import annotations

import numpy as np
import pytest

from general_ai_compiler_b200 import (BackendError, DeviceUnavailableError, Graph, Node, ShapeInferenceError,
                                      TensorSpec, ValidationError, evaluate_op, infer_node)
from general_ai_compiler_b200.bevformer import (WORKLOADS, build_dcn_graph_for, build_msda_graph,
                                                build_msda_graph_for, make_msda_inputs, make_workload_inputs)
from general_ai_compiler_b200.compiler import CudaProgram, compile_cuda, msda_rows_per_cta
from general_ai_compiler_b200.session import CudaSession
from general_ai_compiler_b200.validation import TensorTolerance, bind_inputs, compare_tensor


def _node(spatial_shapes) -> Node:
    return Node("msda", "MSDeformableAttention", ("value", "sampling_locations", "attention_weights"),
                ("output",), {"spatial_shapes": spatial_shapes})


def _specs(*, value=(2, 20, 8, 32), locations=(2, 11, 8, 2, 4, 2), weights=(2, 11, 8, 2, 4), dtype="float32"):
    return {"value": TensorSpec(value, dtype), "sampling_locations": TensorSpec(locations, dtype),
            "attention_weights": TensorSpec(weights, dtype)}


def test_msda_shape_inference():
    assert infer_node(_node([[4, 4], [2, 2]]), _specs()) == {"output": TensorSpec((2, 11, 256), "float32")}
    assert infer_node(_node([[4, 4], [2, 2]]), _specs(dtype="float16"))["output"].dtype == "float16"


@pytest.mark.parametrize("specs,shapes", [
    (_specs(value=(2, 20, 256)), [[4, 4], [2, 2]]),                   # value rank
    (_specs(locations=(2, 11, 8, 8, 2)), [[4, 4], [2, 2]]),           # locations rank
    (_specs(weights=(2, 11, 8, 8)), [[4, 4], [2, 2]]),                # weights rank
    (_specs(locations=(2, 11, 8, 2, 4, 3)), [[4, 4], [2, 2]]),        # coordinate size
    (_specs(locations=(1, 11, 8, 2, 4, 2)), [[4, 4], [2, 2]]),        # batch mismatch
    (_specs(weights=(2, 12, 8, 2, 4)), [[4, 4], [2, 2]]),             # query mismatch
    (_specs(locations=(2, 11, 4, 2, 4, 2)), [[4, 4], [2, 2]]),        # head mismatch
    (_specs(locations=(2, 11, 8, 1, 4, 2)), [[4, 4], [2, 2]]),        # level mismatch
    (_specs(weights=(2, 11, 8, 2, 3)), [[4, 4], [2, 2]]),             # point mismatch
    (_specs(value=(2, 19, 8, 32)), [[4, 4], [2, 2]]),                 # flattened value size
    (_specs(), [[4], [2, 2]]),                                        # malformed spatial shape
    (_specs(), [[4, 4], [0, 2]]),                                     # non-positive spatial shape
    (_specs(dtype="int32"), [[4, 4], [2, 2]]),                        # non-floating value
])
def test_msda_shape_inference_rejects_malformed_contract(specs, shapes):
    with pytest.raises(ShapeInferenceError):
        infer_node(_node(shapes), specs)


def test_fused_offsets_shape_inference():
    node = Node("m", "MSDeformableAttentionOffsets", ("v", "o", "w", "n", "r"), ("y",),
                {"spatial_shapes": [[2, 3], [1, 2]], "coordinate_shape": [2, 3, 2, 2, 2, 2, 2], "reference_first": 1})
    specs = {"v": TensorSpec((2, 8, 2, 3), "float32"), "o": TensorSpec((2, 3, 2, 2, 4, 2), "float32"),
             "w": TensorSpec((2, 3, 2, 2, 4), "float32"), "n": TensorSpec((1, 1, 1, 2, 1, 2), "float32"),
             "r": TensorSpec((2, 3, 1, 1, 1, 2, 2), "float32")}
    assert infer_node(node, specs) == {"y": TensorSpec((2, 3, 6), "float32")}
    bad = dict(specs, r=TensorSpec((2, 3, 1, 1, 1, 3, 2), "float32"))
    with pytest.raises(ShapeInferenceError):
        infer_node(node, bad)


def _dcn_node(**attrs):
    base = {"stride": [1, 1], "padding": [1, 1], "dilation": [1, 1], "groups": 1, "deform_groups": 1}
    base.update(attrs)
    return Node("dcn", "DeformConv2D", ("X", "offset", "mask", "W", "bias"), ("Y",), base)


def _dcn_specs(cin=4, cout=6, h=5, w=6, k=(3, 3), oh=5, ow=6, groups=1, dg=1):
    return {"X": TensorSpec((2, cin, h, w), "float32"), "offset": TensorSpec((2, 2 * dg * k[0] * k[1], oh, ow), "float32"),
            "mask": TensorSpec((2, dg * k[0] * k[1], oh, ow), "float32"),
            "W": TensorSpec((cout, cin // groups, *k), "float32"), "bias": TensorSpec((cout,), "float32")}


def test_dcn_shape_inference():
    assert infer_node(_dcn_node(), _dcn_specs())["Y"].shape == (2, 6, 5, 6)
    # stride 2 / dilation 2 on one axis (the dcn_batch_grouped recipe)
    node = _dcn_node(stride=[2, 1], padding=[1, 0], dilation=[2, 1], groups=2, deform_groups=2)
    specs = _dcn_specs(cin=4, cout=6, h=6, w=7, k=(2, 3), oh=3, ow=5, groups=2, dg=2)
    assert infer_node(node, specs)["Y"].shape == (2, 6, 3, 5)


def test_dcn_shape_inference_rejections():
    with pytest.raises(ShapeInferenceError, match="divisib"):
        infer_node(_dcn_node(groups=3), _dcn_specs())
    bad = _dcn_specs()
    bad["offset"] = TensorSpec((2, 17, 5, 6), "float32")
    with pytest.raises(ShapeInferenceError, match="offset|channels"):
        infer_node(_dcn_node(), bad)
    with pytest.raises(ShapeInferenceError, match="FP32"):
        infer_node(_dcn_node(), {k: TensorSpec(v.shape, "float16") for k, v in _dcn_specs().items()})
    with pytest.raises(ShapeInferenceError, match="exceeds"):
        infer_node(_dcn_node(padding=[0, 0]), _dcn_specs(h=2, w=2, oh=0, ow=0))
    with pytest.raises(ShapeInferenceError):
        infer_node(_dcn_node(stride=[0, 1]), _dcn_specs())


def test_conv2d_shape_inference_follows_the_reference_contract():
    """src/gac/core/ops.py:615-645: four pads (top, left, bottom, right), floor division, divisibility by groups."""
    node = Node("c", "Conv2D", ("X", "W", "b"), ("Y",), {"strides": [2, 1], "pads": [1, 2, 0, 1], "dilations": [1, 2], "groups": 2})
    specs = {"X": TensorSpec((2, 6, 7, 9), "float32"), "W": TensorSpec((8, 3, 3, 3), "float32"), "b": TensorSpec((8,), "float32")}
    assert infer_node(node, specs)["Y"].shape == (2, 8, 3, 8)
    plain = Node("c", "Conv2D", ("X", "W"), ("Y",), {})
    assert infer_node(plain, {"X": TensorSpec((1, 256, 58, 100), "float32"), "W": TensorSpec((27, 256, 3, 3), "float32")})["Y"].shape == (1, 27, 56, 98)
    with pytest.raises(ShapeInferenceError, match="groups"):
        infer_node(Node("c", "Conv2D", ("X", "W"), ("Y",), {"groups": 4}), specs)
    with pytest.raises(ShapeInferenceError, match="bias"):
        infer_node(node, {**specs, "b": TensorSpec((7,), "float32")})
    with pytest.raises(ShapeInferenceError, match="pads"):
        infer_node(Node("c", "Conv2D", ("X", "W"), ("Y",), {"pads": [1, 1]}), specs)
    with pytest.raises(ShapeInferenceError, match="non-positive"):
        infer_node(plain, {"X": TensorSpec((1, 3, 2, 2), "float32"), "W": TensorSpec((4, 3, 3, 3), "float32")})
    with pytest.raises(ShapeInferenceError, match="FP32"):
        infer_node(plain, {"X": TensorSpec((1, 3, 5, 5), "float16"), "W": TensorSpec((4, 3, 3, 3), "float16")})


def test_graph_validation_and_json_round_trip():
    g = build_msda_graph()
    g.validate()
    again = Graph.from_json(g.to_json())
    assert again.inputs == g.inputs and again.outputs == g.outputs
    assert again.nodes[0].attrs["spatial_shapes"] == [[15, 25]]
    with pytest.raises(ValidationError):
        Graph("bad", {"a": TensorSpec((1,), "float32")}, ("missing",), []).validate()
    with pytest.raises(ValidationError):
        Graph("bad", {"a": TensorSpec((1,), "float32")}, ("b",),
              [Node("n", "X", ("later",), ("b",))]).validate()
    with pytest.raises(ValidationError):
        TensorSpec((-1,), "float32")
    with pytest.raises(ValidationError):
        Node("", "op", (), ("y",))


def test_tiny_profile_graph_and_inputs():
    g = build_msda_graph()
    assert g.inputs == {"value": TensorSpec((6, 375, 8, 32), "float32"),
                        "sampling_locations": TensorSpec((6, 2500, 8, 1, 8, 2), "float32"),
                        "attention_weights": TensorSpec((6, 2500, 8, 1, 8), "float32")}
    assert g.value_specs["output"] == TensorSpec((6, 2500, 256), "float32")
    a, b = make_msda_inputs(g, seed=20261010), make_msda_inputs(g, seed=20261010)
    for name, arr in a.items():
        assert arr.flags.c_contiguous and arr.dtype == np.float32 and np.all(np.isfinite(arr))
        assert np.array_equal(arr, b[name])
    np.testing.assert_allclose(a["attention_weights"].sum(axis=(3, 4)), np.ones((6, 2500, 8), np.float32),
                               rtol=1e-6, atol=1e-6)
    with pytest.raises(ValidationError):
        make_msda_inputs(g, seed=True)


def test_workload_inputs_follow_the_stated_distributions():
    w = WORKLOADS["tiny_tsa"]
    x = make_workload_inputs(w)
    loc = x["sampling_locations"]
    assert loc.shape == (2, 2500, 8, 1, 4, 2) and loc.min() >= -0.05 and loc.max() <= 1.05
    outside = float(((loc < 0) | (loc > 1)).mean())
    assert 0.05 < outside < 0.13
    np.testing.assert_allclose(x["attention_weights"].sum(axis=(3, 4)), 1.0, rtol=1e-5)
    w = WORKLOADS["base_tsa"].with_queries(400)
    loc = make_workload_inputs(w)["sampling_locations"]
    centre = loc.mean(axis=(0, 2, 3, 4))
    np.testing.assert_allclose(centre[0], [0.025, 0.025], atol=0.01)
    np.testing.assert_allclose(centre[21], [0.075, 0.075], atol=0.01)   # second BEV row, x fastest
    assert WORKLOADS["base_sca"].samples == 15_360_000
    assert WORKLOADS["base_sca"].algorithmic_bytes(4) == 435_148_800
    assert WORKLOADS["dcn_c4"].flops == WORKLOADS["dcn_c5"].flops == 41_051_750_400
    d = make_workload_inputs(WORKLOADS["dcn_c5"])
    assert d["X"].shape == (6, 512, 29, 50) and d["offset"].shape == (6, 18, 29, 50) and d["mask"].shape == (6, 9, 29, 50)
    assert 0 < d["mask"].min() and d["mask"].max() < 1 and abs(float(d["offset"].std()) - np.sqrt(2)) < 0.02


def test_compile_plans_one_launch_per_node():
    first, second = compile_cuda(build_msda_graph()), compile_cuda(build_msda_graph())
    assert isinstance(first, CudaProgram) and first.source == second.source
    assert len(first.launches) == 1
    launch = first.launches[0]
    assert launch.node_id == "msda" and launch.entry_point == "gacb_msda_forward"
    # the launch metadata is what the library launches (gacb_msda_launch_geometry): float32 texels run thread
    # blocks of 128 threads, 16 rows side by side; 6*2500*8 rows with 8 samples each take two row batches per block
    assert launch.block == (128, 1, 1) and launch.implementation_candidates == ("msda_rows_kernel<float,4,8>",)
    assert msda_rows_per_cta(32, 8) == 32 and launch.grid == (6 * 2500 * 8 // 32, 1, 1)
    assert msda_rows_per_cta(32, 8, "bfloat16") == 64 and msda_rows_per_cta(6, 8) is None
    assert first.describe()["tensor_bytes_upper_bound"] == 29_184_000
    base = compile_cuda(build_msda_graph_for(WORKLOADS["base_sca"]))
    assert base.launches[0].grid == (30000, 1, 1) and base.launches[0].block == (128, 1, 1)
    bf16 = compile_cuda(build_msda_graph_for(WORKLOADS["base_sca"]), value_storage="bfloat16")
    assert bf16.launches[0].grid == (7500, 1, 1) and bf16.launches[0].block == (256, 1, 1)
    dcn = compile_cuda(build_dcn_graph_for(WORKLOADS["dcn_c4"]), dcn_math="bf16")
    assert dcn.launches[0].entry_point == "gacb_dcnv2_forward" and dcn.options["dcn_math"] == "bf16"
    # 6 * 58 * 100 output pixels in tiles of 128, one 256-channel tile, 19 warps per thread block
    assert dcn.launches[0].grid == (272, 1, 1) and dcn.launches[0].block == (608, 1, 1)
    assert dcn.launches[0].implementation_candidates == ("dcn_umma_kernel<bf16,deform,wide>",)
    assert "3xTF32" not in first.describe()["precision"]


def test_launch_geometry_follows_the_kernel_dispatch_rules():
    """What compile_cuda reports is computed by the same planning code that launches: spot checks of its rules."""
    from general_ai_compiler_b200 import native

    tiny = native.dcnv2_launch_geometry(1, 8, 5, 5, 8, 3, 3, (1, 1), (1, 1), (1, 1), 1, 1, native.DCN_BF16)
    assert tiny.kernel == b"dcn_direct_kernel" and tuple(tiny.block) == (256, 1, 1) and tuple(tiny.grid) == (1, 1, 1)
    # conv_offset: the persistent window kernel in every math mode, one CTA per SM over 6 * 13 * 4 tiles of 16 x 8 pixels
    # (tensor copies bring the windows in BF16 and TF32 mode: 10 warps; F32X3 launches eight fill warps more)
    for mode, name, threads in ((native.DCN_BF16, b"bf16", 320), (native.DCN_TF32, b"tf32", 320), (native.DCN_F32X3, b"f32x3", 544)):
        conv = native.dcnv2_launch_geometry(6, 256, 58, 100, 27, 3, 3, (1, 1), (1, 1), (1, 1), 1, 1, mode, plain=True)
        assert conv.kernel == b"conv_window_kernel<" + name + b">" and tuple(conv.block) == (threads, 1, 1)
        assert tuple(conv.grid) == (148, 1, 1) and conv.dynamic_smem_bytes <= 227 * 1024
    few = native.dcnv2_launch_geometry(1, 256, 58, 100, 27, 3, 3, (1, 1), (1, 1), (1, 1), 1, 1, native.DCN_BF16, plain=True)
    assert few.kernel == b"conv_window_kernel<bf16>" and tuple(few.grid) == (52, 1, 1)
    # what does not qualify keeps the gather kernel: two CTAs per SM beyond one wave, the wide shape within one wave
    conv = native.dcnv2_launch_geometry(6, 256, 58, 100, 27, 3, 3, (1, 1), (2, 2), (2, 2), 1, 1, native.DCN_TF32, plain=True)
    assert conv.kernel == b"dcn_umma_kernel<tf32,plain,narrow>" and tuple(conv.block) == (352, 1, 1)
    one_wave = native.dcnv2_launch_geometry(3, 256, 58, 100, 27, 3, 3, (1, 1), (2, 2), (2, 2), 1, 1, native.DCN_TF32, plain=True)
    assert one_wave.kernel == b"dcn_umma_kernel<tf32,plain,wide>" and tuple(one_wave.grid) == (136, 1, 1)
    wide_out = native.dcnv2_launch_geometry(6, 256, 58, 100, 48, 3, 3, (1, 1), (1, 1), (1, 1), 1, 1, native.DCN_F32X3, plain=True)
    assert wide_out.kernel.startswith(b"dcn_umma_kernel<f32x3,plain")       # F32X3 windows stop at 32 output channels
    c5 = native.dcnv2_launch_geometry(6, 512, 29, 50, 512, 3, 3, (1, 1), (1, 1), (1, 1), 1, 1, native.DCN_F32X3)
    assert tuple(c5.grid) == (68, 2, 1) and c5.dynamic_smem_bytes <= 227 * 1024
    odd = native.msda_launch_geometry(native.GACB_F32, [(3, 5)], 2, 7, 3, 6, 2)
    assert odd.kernel == b"msda_generic_kernel" and tuple(odd.block) == (256, 1, 1) and odd.grid[0] == 1
    part = native.msda_launch_geometry(native.GACB_F32, [(116, 200), (58, 100), (29, 50), (15, 25)], 6, 10000, 8, 32, 8,
                                       q_range=(1250, 2500))
    assert part.grid[0] == 6 * 1250 * 8 // 16 and part.units_per_cta == 16


def test_backend_rejects_non_float32_and_unknown_ops():
    g = Graph("msda_fp16", {"value": TensorSpec((1, 1, 1, 1), "float16"),
                            "sampling_locations": TensorSpec((1, 1, 1, 1, 1, 2), "float16"),
                            "attention_weights": TensorSpec((1, 1, 1, 1, 1), "float16")}, ("output",),
              [_node([[1, 1]])])
    with pytest.raises(BackendError):
        compile_cuda(g)
    other = Graph("relu", {"x": TensorSpec((1,), "float32")}, ("y",), [Node("r", "Relu", ("x",), ("y",))])
    with pytest.raises(BackendError):
        compile_cuda(other)
    many = Graph("levels", {"value": TensorSpec((1, 33, 1, 4), "float32"),
                            "sampling_locations": TensorSpec((1, 1, 1, 33, 1, 2), "float32"),
                            "attention_weights": TensorSpec((1, 1, 1, 33, 1), "float32")}, ("output",),
                 [_node([[1, 1]] * 33)])
    with pytest.raises(BackendError, match="levels"):
        compile_cuda(many)


def test_bind_inputs_enforces_the_graph_abi():
    g = build_msda_graph_for(WORKLOADS["tiny_sca"].with_queries(4))
    x = make_workload_inputs(WORKLOADS["tiny_sca"].with_queries(4))
    assert set(bind_inputs(g, x)) == set(g.inputs)
    with pytest.raises(ValidationError, match="names"):
        bind_inputs(g, {"value": x["value"]})
    with pytest.raises(ValidationError, match="requires"):
        bind_inputs(g, dict(x, value=x["value"].astype(np.float64)))
    with pytest.raises(ValidationError, match="contiguous"):
        bind_inputs(g, dict(x, value=np.asfortranarray(x["value"])))
    bad = x["value"].copy()
    bad[0, 0, 0, 0] = np.nan
    with pytest.raises(ValidationError, match="finite"):
        bind_inputs(g, dict(x, value=bad))


def test_checked_copy_copies_and_finds_non_finite_values_in_one_pass():
    from general_ai_compiler_b200.validation import checked_copy

    rng = np.random.default_rng(3)
    for shape in ((7,), (3, 1000, 33), (6, 1 << 20)):          # below and above the pooled size
        src = rng.standard_normal(shape).astype(np.float32)
        dst = np.full(shape, 7.0, np.float32)
        checked_copy(dst, src, "x")
        assert np.array_equal(dst, src)
        for bad in (np.nan, np.inf, -np.inf):
            poisoned = src.copy()
            poisoned.reshape(-1)[poisoned.size - 2] = bad
            with pytest.raises(ValidationError, match="input 'x' must contain finite values"):
                checked_copy(dst, poisoned, "x")
    # a destination that is not contiguous still gets the values
    wide = np.zeros((4, 10), np.float32)
    checked_copy(wide[:, ::2], np.ones((4, 5), np.float32), "y")
    assert wide[:, ::2].sum() == 20 and wide[:, 1::2].sum() == 0


def test_compare_tensor_metrics():
    ref = np.linspace(-1, 1, 101, dtype=np.float32)
    same = compare_tensor(ref, ref)
    assert same.passed and same.max_abs == 0 and same.cosine == 1.0 and same.close_fraction == 1.0
    off = compare_tensor(ref + np.float32(3e-4), ref)
    assert not off.passed and off.close_fraction < 1.0
    assert compare_tensor(ref + np.float32(3e-4), ref, TensorTolerance(rtol=0, atol=1e-3)).passed
    with pytest.raises(ValidationError):
        compare_tensor(ref[:-1], ref)


def test_no_cpu_fallback_without_a_device():
    """Without a GPU every execution entry raises; nothing is computed on the host."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    w = WORKLOADS["tiny_sca"].with_queries(2)
    x = make_workload_inputs(w)
    with pytest.raises(DeviceUnavailableError):
        evaluate_op("MSDeformableAttention", (x["value"], x["sampling_locations"], x["attention_weights"]),
                    {"spatial_shapes": w.spatial_shapes})
    with pytest.raises(DeviceUnavailableError):
        CudaSession(compile_cuda(build_msda_graph_for(w)))
