"""The graph pass that folds BEVFormer's neighbours into the sampling launches, and the fused launches themselves."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import assert_fp32_gate
from general_ai_compiler_b200.bevformer import (DcnWorkload, build_dcn_block_graph, build_dcn_bottleneck_graph,
                                                build_sca_block_graph, build_tsa_tail_graph, make_workload_inputs)
from general_ai_compiler_b200.compiler import compile_cuda
from general_ai_compiler_b200.errors import BackendError
from general_ai_compiler_b200.ir import Graph, Node, TensorSpec
from general_ai_compiler_b200.passes import FUSED_MSDA, fuse_deformable_sampling

SCA = dict(samples=1, cameras=3, queries=40, heads=8, head_dim=32, spatial_shapes=[(12, 20), (6, 10)],
           points_per_anchor=2, anchors=4)


def test_sca_block_becomes_one_launch():
    g = build_sca_block_graph(**SCA)
    fused, report = fuse_deformable_sampling(g)
    assert report["changed"] and report["details"]["fused"][0]["fused"] == ["softmax", "coordinates", "camera average"]
    assert len(g.nodes) == 18 and [n.op for n in fused.nodes] == ["Reshape", "Reshape", "Reshape", FUSED_MSDA]
    node = fused.nodes[-1]
    assert node.inputs == ("value_msda", "offset_flat", "attention_flat", "offset_normalizer", "reference_nq111a2", "visibility")
    a = node.attrs
    assert a["softmax"] and a["coordinates"] == "offsets" and a["reduce"] == "masked_average" and a["group"] == 3
    assert a["coordinate_shape"] == [3, 40, 8, 2, 2, 4, 2] and a["reference_first"] is True
    assert a["normalizer_shape"] == [1, 1, 1, 2, 1, 2] and a["reference_shape"] == [3, 40, 1, 1, 1, 4, 2]
    program = compile_cuda(g)
    assert [l.entry_point for l in program.launches] == ["gacb_msda_run"]
    assert program.graph.value_specs["averaged_context"].shape == (1, 40, 256)
    assert len(program.reference_graph.nodes) == 18                      # the graph as given is kept beside it
    assert "spatial_msda" in program.launches[0].source_nodes or program.launches[0].source_nodes
    with pytest.raises(BackendError, match="outside"):
        compile_cuda(g, fuse=False)                                      # unfused, Softmax & co. are not this backend's


def test_patterns_that_do_not_match_are_left_alone():
    g = build_sca_block_graph(**SCA)
    # the probabilities are also a graph output: the softmax must stay a node (and then the graph is not ours)
    exposed = Graph(g.name, g.inputs, ("averaged_context", "attention_probability"), g.nodes, g.constants)
    fused, report = fuse_deformable_sampling(exposed)
    kinds = report["details"]["fused"][0]["fused"]
    assert "softmax" not in kinds and "coordinates" in kinds and "camera average" in kinds
    assert any(n.op == "Softmax" for n in fused.nodes)
    # a clamp with another floor is not the visible-count guard
    nodes = [Node(n.id, n.op, n.inputs, n.outputs, {"min": 2.0}) if n.id == "visibility_clamp" else n for n in g.nodes]
    fused, report = fuse_deformable_sampling(Graph(g.name, g.inputs, g.outputs, nodes, g.constants))
    assert "camera average" not in report["details"]["fused"][0]["fused"]
    assert any(n.op == "Clamp" for n in fused.nodes)
    # softmax over another axis
    nodes = [Node(n.id, n.op, n.inputs, n.outputs, {"axis": 1}) if n.id == "attention_softmax" else n for n in g.nodes]
    _, report = fuse_deformable_sampling(Graph(g.name, g.inputs, g.outputs, nodes, g.constants))
    assert "softmax" not in report["details"]["fused"][0]["fused"]
    # a normaliser that varies along one of the two merged point axes cannot be expressed against [B,Q,H,L,P,2]
    bad = g.constants["offset_normalizer"] * np.ones((1, 1, 1, 1, 2, 1, 1), np.float32)
    _, report = fuse_deformable_sampling(Graph(g.name, g.inputs, g.outputs, g.nodes, {"offset_normalizer": bad}))
    assert "coordinates" not in report["details"]["fused"][0]["fused"]


def test_tsa_tail_and_dcn_block():
    program = compile_cuda(build_tsa_tail_graph(1, 2, 50, 8, 32, (10, 10), 4))
    (node,) = program.graph.nodes
    assert node.op == FUSED_MSDA and node.attrs["reduce"] == "mean" and node.attrs["group"] == 2
    assert program.graph.value_specs["context"].shape == (1, 50, 256)
    program = compile_cuda(build_dcn_block_graph(DcnWorkload("b", 1, 64, 10, 12, 64)))
    (node,) = program.graph.nodes
    assert node.op == "DeformConv2D" and len(node.inputs) == 9 and node.inputs[2] == "mask_scores"
    assert node.attrs["mask_is_logits"] and node.attrs["batch_norm"] and node.attrs["relu"] and node.outputs == ("Y",)
    # Conv2D -> ReLU, GAC's own fusion (native/lib/GraphPasses.cpp:338-341)
    g = Graph("c", {"X": TensorSpec((1, 8, 6, 6), "float32"), "W": TensorSpec((4, 8, 3, 3), "float32")}, ("Y",),
              [Node("conv", "Conv2D", ("X", "W"), ("T",), {"pads": [1, 1, 1, 1]}), Node("act", "ReLU", ("T",), ("Y",))])
    (node,) = compile_cuda(g).graph.nodes
    assert node.op == "Conv2D" and node.attrs["relu"] and node.outputs == ("Y",)


# --------------------------------------------------------------------------- GPU

def _sca_inputs(seed=3):
    rng = np.random.default_rng(seed)
    s = SCA
    n, q, h = s["samples"] * s["cameras"], s["queries"], s["heads"]
    levels, points = len(s["spatial_shapes"]), s["points_per_anchor"] * s["anchors"]
    spatial = sum(a * b for a, b in s["spatial_shapes"])
    return {
        "value_projected": rng.standard_normal((n, spatial, h * s["head_dim"])).astype(np.float32),
        "offset_flat": (rng.standard_normal((n, q, h * levels * points * 2)) * 1.5).astype(np.float32),
        "reference_points": rng.uniform(-0.05, 1.05, (s["samples"], s["cameras"], q, s["anchors"], 2)).astype(np.float32),
        "attention_flat": rng.standard_normal((n, q, h * levels * points)).astype(np.float32),
        "visibility": (rng.random((s["samples"], s["cameras"], q, 1)) < 0.6).astype(np.float32),
    }


@pytest.mark.gpu
@pytest.mark.parametrize("storage", ["float32", "bfloat16"])
def test_fused_sca_block_matches_the_unfused_operators(storage):
    """Expected value: the oracle's operators applied one after the other, as the reference evaluates the graph."""
    from conftest import assert_rel_gate
    from general_ai_compiler_b200.session import CudaSession
    from oracle.msda_numpy import msda_offsets_forward, sca_camera_average, softmax_last

    g = build_sca_block_graph(**SCA)
    x = _sca_inputs()
    s = SCA
    n, q, h = s["samples"] * s["cameras"], s["queries"], s["heads"]
    levels, points = len(s["spatial_shapes"]), s["points_per_anchor"] * s["anchors"]
    coord = (n, q, h, levels, s["points_per_anchor"], s["anchors"], 2)
    value = x["value_projected"].reshape(n, -1, h, s["head_dim"])
    weights = softmax_last(x["attention_flat"].reshape(n, q, h, levels * points)).reshape(n, q, h, levels, points).astype(np.float32)
    per_camera = msda_offsets_forward(value, x["offset_flat"].reshape(n, q, h, levels, points, 2), weights,
                                      g.constants["offset_normalizer"].reshape(1, 1, 1, levels, 1, 2),
                                      x["reference_points"].reshape(n, q, 1, 1, 1, s["anchors"], 2), s["spatial_shapes"],
                                      coord, reference_first=True)
    want = sca_camera_average(per_camera, x["visibility"], s["cameras"])
    with CudaSession(compile_cuda(g, value_storage=storage)) as session:
        got = session.run(x).outputs["averaged_context"]
        again = session.run(x).outputs["averaged_context"]
    assert got.shape == (1, q, 256) and np.array_equal(got, again)
    if storage == "float32":
        assert_fp32_gate(got, want, "fused SCA block")
    else:
        assert_rel_gate(got, want, 1e-2, "fused SCA block, bf16 value")


@pytest.mark.gpu
def test_fused_tsa_tail_and_dcn_block_match_the_unfused_operators():
    from general_ai_compiler_b200.session import CudaSession
    from oracle import dcnv2_fused_c
    from oracle.msda_numpy import msda_forward, tsa_queue_mean

    rng = np.random.default_rng(8)
    g = build_tsa_tail_graph(2, 2, 60, 8, 32, (12, 9), 4)
    x = {"value_msda": rng.standard_normal((4, 108, 8, 32)).astype(np.float32),
         "sampling_locations": rng.uniform(-0.1, 1.1, (4, 60, 8, 1, 4, 2)).astype(np.float32),
         "attention_weights": rng.random((4, 60, 8, 1, 4)).astype(np.float32)}
    want = tsa_queue_mean(msda_forward(x["value_msda"], x["sampling_locations"], x["attention_weights"], [(12, 9)]), 2)
    with CudaSession(compile_cuda(g)) as session:
        assert_fp32_gate(session.run(x).outputs["context"], want, "fused TSA tail")

    wl = DcnWorkload("blk", 2, 64, 20, 24, 64, seed=5)
    base = make_workload_inputs(wl)
    x = {"X": base["X"], "offset": base["offset"], "mask_scores": (rng.standard_normal(base["mask"].shape) * 2).astype(np.float32),
         "W": base["W"], "bias": base["bias"], "bn_scale": rng.uniform(0.5, 1.5, 64).astype(np.float32),
         "bn_bias": rng.standard_normal(64).astype(np.float32), "bn_mean": (rng.standard_normal(64) * 0.2).astype(np.float32),
         "bn_variance": rng.uniform(0.3, 2.0, 64).astype(np.float32)}
    want = dcnv2_fused_c(x["X"], x["offset"], x["mask_scores"], x["W"], x["bias"],
                         bn=(x["bn_scale"], x["bn_bias"], x["bn_mean"], x["bn_variance"], 1e-5), relu=True,
                         stride=(1, 1), padding=(1, 1), dilation=(1, 1))
    with CudaSession(compile_cuda(build_dcn_block_graph(wl))) as session:
        assert_fp32_gate(session.run(x).outputs["Y"], want, "fused DCN block")


def _bottleneck_constants(wl, seed=3):
    rng = np.random.default_rng(seed)
    base = make_workload_inputs(wl)
    k3 = 3 * wl.kernel[0] * wl.kernel[1]
    return {"W_offset": (rng.standard_normal((k3, wl.cin, *wl.kernel)) * 0.02).astype(np.float32),
            "b_offset": (rng.standard_normal(k3) * 0.1).astype(np.float32), "W": base["W"], "bias": base["bias"],
            "bn_scale": rng.uniform(0.5, 1.5, wl.cout).astype(np.float32), "bn_bias": rng.standard_normal(wl.cout).astype(np.float32),
            "bn_mean": (rng.standard_normal(wl.cout) * 0.2).astype(np.float32),
            "bn_variance": rng.uniform(0.3, 2.0, wl.cout).astype(np.float32)}, base["X"]


@pytest.mark.parametrize("three_way", [False, True])
def test_bottleneck_becomes_two_launches(three_way):
    """conv_offset -> Slice (-> Concat) -> Sigmoid -> DeformConv2D -> BatchNorm -> ReLU: the convolution writes the
    offsets and the mask scores as two tensors, the DCNv2 takes the sigmoid, the normalisation and the ReLU."""
    wl = DcnWorkload("neck", 2, 64, 20, 24, 64, seed=5)
    constants, _ = _bottleneck_constants(wl)
    g = build_dcn_bottleneck_graph(wl, constants, three_way=three_way)
    fused, report = fuse_deformable_sampling(g)
    assert report["changed"] and [n.op for n in fused.nodes] == ["Conv2D", "DeformConv2D"]
    conv, dcn = fused.nodes
    assert conv.attrs["split_at"] == 18 and conv.outputs == ("offset", "mask_scores")
    assert dcn.inputs[:3] == ("X", "offset", "mask_scores") and dcn.attrs["mask_is_logits"] and dcn.attrs["batch_norm"]
    assert dcn.attrs["relu"] and dcn.outputs == ("Y",)
    assert fused.value_specs["offset"].shape == (2, 18, 20, 24) and fused.value_specs["mask_scores"].shape == (2, 9, 20, 24)
    kinds = {d["node"]: d["fused"] for d in report["details"]["fused"]}
    assert kinds == {"conv_offset": ["channel split"], "conv2": ["sigmoid", "batch norm", "relu"]}
    program = compile_cuda(g)
    assert [l.entry_point for l in program.launches] == ["gacb_conv2d_forward", "gacb_dcnv2_fused_forward"] or \
        [l.entry_point for l in program.launches] == ["gacb_conv2d_forward", "gacb_dcnv2_forward"]
    assert program.launches[0].output == "offset" and program.launches[0].extra_outputs == ("mask_scores",)
    # a convolution output that something else reads as well, or that the graph exposes, stays whole
    nodes = list(g.nodes) + [Node("also_reads", "ReLU", ("offset_mask",), ("side",))]
    _, report = fuse_deformable_sampling(Graph(g.name, g.inputs, ("Y", "side"), nodes, g.constants))
    assert all("channel split" not in d["fused"] for d in report["details"]["fused"])
    exposed = Graph(g.name, g.inputs, ("Y", "offset_mask"), g.nodes, g.constants)
    _, report = fuse_deformable_sampling(exposed)
    assert all("channel split" not in d["fused"] for d in report["details"]["fused"])


@pytest.mark.gpu
@pytest.mark.parametrize("math", ["f32x3", "bf16"])
def test_bottleneck_session_matches_the_operator_chain(math):
    """The session's two launches against the same two operators called by hand (bit-identical: same kernels), and
    against the C oracle's chain at the gate the chain test uses (an offset that differs in the last bit moves a
    sample across a texel)."""
    import torch

    from general_ai_compiler_b200 import ops
    from general_ai_compiler_b200.session import CudaSession
    from oracle import conv2d_c, dcnv2_fused_c

    wl = DcnWorkload("neck", 2, 64, 40, 36, 64, seed=6)
    constants, x = _bottleneck_constants(wl, seed=4)
    g = build_dcn_bottleneck_graph(wl, constants, three_way=True)
    with CudaSession(compile_cuda(g, dcn_math=math)) as session:
        assert session._input_copy == {"conv_offset": "make", "conv2": "reuse"}
        first = session.run({"X": x}).outputs["Y"]
        again = session.run({"X": x}).outputs["Y"]            # packed weights reused
    assert np.array_equal(first, again)
    device = ops.require_device(0)
    t = {k: torch.from_numpy(v).to(device) for k, v in {**constants, "X": x}.items()}
    off, scores = ops.conv2d_forward(t["X"], t["W_offset"], t["b_offset"], pads=(1, 1, 1, 1), math=math, split_at=18)
    y = ops.dcnv2_forward(t["X"], off, scores, t["W"], t["bias"], stride=wl.stride, padding=wl.padding, dilation=wl.dilation,
                          math=math, mask_is_logits=True, relu=True,
                          batch_norm=(t["bn_scale"], t["bn_bias"], t["bn_mean"], t["bn_variance"], 1e-5))
    assert np.array_equal(first, y.cpu().numpy())
    om = conv2d_c(x, constants["W_offset"], constants["b_offset"], pads=(1, 1, 1, 1))
    want = dcnv2_fused_c(x, np.ascontiguousarray(om[:, :18]), np.ascontiguousarray(om[:, 18:]), constants["W"], constants["bias"],
                         bn=(constants["bn_scale"], constants["bn_bias"], constants["bn_mean"], constants["bn_variance"], 1e-5),
                         relu=True, stride=wl.stride, padding=wl.padding, dilation=wl.dilation)
    scale = float(np.abs(want).max())
    assert float(np.abs(first - want).max()) <= (1e-3 if math == "f32x3" else 2e-2) * scale


@pytest.mark.gpu
def test_cuda_graph_replay_matches_launch_by_launch():
    """A session that replays its launch sequence as a CUDA graph returns, run after run and for new inputs, exactly
    what the launch-by-launch session returns."""
    from general_ai_compiler_b200.session import CudaSession

    rng = np.random.default_rng(21)
    wl = DcnWorkload("blk", 2, 64, 20, 24, 64, seed=6)
    base = make_workload_inputs(wl)

    def dcn_inputs():
        return {"X": rng.standard_normal(base["X"].shape).astype(np.float32), "offset": base["offset"],
                "mask_scores": (rng.standard_normal(base["mask"].shape) * 2).astype(np.float32), "W": base["W"],
                "bias": base["bias"], "bn_scale": rng.uniform(0.5, 1.5, 64).astype(np.float32),
                "bn_bias": rng.standard_normal(64).astype(np.float32),
                "bn_mean": (rng.standard_normal(64) * 0.2).astype(np.float32),
                "bn_variance": rng.uniform(0.3, 2.0, 64).astype(np.float32)}

    cases = [(build_sca_block_graph(**SCA), lambda: _sca_inputs(int(rng.integers(1 << 30))), "averaged_context"),
             (build_dcn_block_graph(wl), dcn_inputs, "Y")]
    for graph, make, name in cases:
        program = compile_cuda(graph)
        with CudaSession(program) as eager, CudaSession(program, cuda_graph=True) as replayed:
            for step in range(4):          # step 0 runs eagerly, step 1 captures, steps 2 and 3 only replay
                x = make()
                want = eager.run(x).outputs[name]
                got = replayed.run(x).outputs[name]
                assert np.array_equal(got, want), f"{graph.name}: step {step}"
            assert replayed._graph is not None
            traced = replayed.run(x, trace=True)      # instrumented runs stay launch by launch
            assert np.array_equal(traced.outputs[name], want) and traced.kernel_ms is not None
