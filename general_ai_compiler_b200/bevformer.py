"""BEVFormer workloads for the deformable-sampling path: graphs and seeded inputs.

``build_msda_graph`` / ``make_msda_inputs`` reproduce the reference's tiny
spatial-cross-attention slice and its input recipe
(``src/gac/models/bevformer/model.py:137-235``): same names, shapes, seed
handling and value distributions, so arrays made here equal the reference's
for the same seed.

``WORKLOADS`` names the five benchmark configurations (synthetic stand-ins with
BEVFormer's shapes; no dataset is involved) and ``make_workload_inputs``
builds their seeded tensors:

==========  =====================================================================
tiny_tsa    value [2,2500,8,32], 50x50, Q=2500, P=4, locations U(-0.05,1.05)
tiny_sca    value [6,375,8,32], 15x25, Q=2500, P=8, reference point + N(0,0.03)
base_sca    value [6,30825,8,32], 4 levels, Q=10000, P=8, reference + N(0,0.02)
base_tsa    value [2,40000,8,32], 200x200, Q=40000, P=4, BEV grid + N(0,0.01)
dcn_c4/c5   DCNv2 3x3 of the R101-DCN stages: X [6,256,58,100] / [6,512,29,50]
==========  =====================================================================
"""

from __future__ import annotations

from dataclasses import dataclass
from numbers import Integral
from typing import Mapping

import numpy as np

from .errors import ValidationError
from .ir import Graph, Node, TensorSpec
from .ops import infer_node


@dataclass(frozen=True)
class MsdaWorkload:
    name: str
    batch: int
    queries: int
    heads: int
    head_dim: int
    points: int
    spatial_shapes: tuple
    location_model: str     # "uniform", "reference_gauss", "bev_grid"
    sigma: float = 0.0
    seed: int = 0

    @property
    def levels(self) -> int:
        return len(self.spatial_shapes)

    @property
    def spatial_size(self) -> int:
        return sum(h * w for h, w in self.spatial_shapes)

    @property
    def samples(self) -> int:
        return self.batch * self.queries * self.heads * self.levels * self.points

    def with_queries(self, queries: int) -> "MsdaWorkload":
        return MsdaWorkload(self.name, self.batch, int(queries), self.heads, self.head_dim, self.points,
                            self.spatial_shapes, self.location_model, self.sigma, self.seed)

    def algorithmic_bytes(self, value_itemsize: int = 4) -> int:
        """Compulsory traffic of one call: value + locations + weights + output, each once."""
        b, q, h, d = self.batch, self.queries, self.heads, self.head_dim
        lp = self.levels * self.points
        return b * self.spatial_size * h * d * value_itemsize + b * q * h * lp * 12 + b * q * h * d * 4


@dataclass(frozen=True)
class DcnWorkload:
    name: str
    batch: int
    cin: int
    height: int
    width: int
    cout: int
    kernel: tuple = (3, 3)
    stride: tuple = (1, 1)
    padding: tuple = (1, 1)
    dilation: tuple = (1, 1)
    groups: int = 1
    deform_groups: int = 1
    seed: int = 0

    @property
    def out_hw(self):
        kh, kw = self.kernel
        ho = (self.height + 2 * self.padding[0] - self.dilation[0] * (kh - 1) - 1) // self.stride[0] + 1
        wo = (self.width + 2 * self.padding[1] - self.dilation[1] * (kw - 1) - 1) // self.stride[1] + 1
        return ho, wo

    @property
    def flops(self) -> int:
        ho, wo = self.out_hw
        return 2 * self.batch * self.cout * (self.cin // self.groups) * self.kernel[0] * self.kernel[1] * ho * wo

    def attrs(self) -> dict:
        return {"stride": list(self.stride), "padding": list(self.padding), "dilation": list(self.dilation),
                "groups": self.groups, "deform_groups": self.deform_groups}


WORKLOADS: Mapping[str, object] = {
    "tiny_tsa": MsdaWorkload("tiny_tsa", 2, 2500, 8, 32, 4, ((50, 50),), "uniform", 0.0, 20261125),
    "tiny_sca": MsdaWorkload("tiny_sca", 6, 2500, 8, 32, 8, ((15, 25),), "reference_gauss", 0.03, 20261126),
    "base_sca": MsdaWorkload("base_sca", 6, 10000, 8, 32, 8, ((116, 200), (58, 100), (29, 50), (15, 25)),
                             "reference_gauss", 0.02, 20261127),
    "base_tsa": MsdaWorkload("base_tsa", 2, 40000, 8, 32, 4, ((200, 200),), "bev_grid", 0.01, 20261128),
    "dcn_c4": DcnWorkload("dcn_c4", 6, 256, 58, 100, 256, seed=20261129),
    "dcn_c5": DcnWorkload("dcn_c5", 6, 512, 29, 50, 512, seed=20261130),
}


def _softmax_last(logits: np.ndarray) -> np.ndarray:
    z = logits - logits.max(axis=-1, keepdims=True)
    e = np.exp(z)
    return (e / e.sum(axis=-1, keepdims=True)).astype(np.float32)


def make_workload_inputs(w, seed: int | None = None) -> dict:
    """Seeded float32, C-contiguous tensors for one workload (deterministic per seed)."""
    rng = np.random.default_rng(w.seed if seed is None else int(seed))
    if isinstance(w, DcnWorkload):
        kh, kw = w.kernel
        ho, wo = w.out_hw
        k = kh * kw
        x = rng.standard_normal((w.batch, w.cin, w.height, w.width), dtype=np.float32)
        cin_g = w.cin // w.groups
        weight = (rng.standard_normal((w.cout, cin_g, kh, kw), dtype=np.float32)
                  * np.float32(np.sqrt(2.0 / (k * cin_g))))
        offset = rng.standard_normal((w.batch, 2 * w.deform_groups * k, ho, wo), dtype=np.float32) * np.float32(np.sqrt(2.0))
        logits = rng.standard_normal((w.batch, w.deform_groups * k, ho, wo), dtype=np.float32)
        mask = (1.0 / (1.0 + np.exp(-logits))).astype(np.float32)
        bias = rng.standard_normal((w.cout,), dtype=np.float32)
        return {"X": x, "offset": np.ascontiguousarray(offset), "mask": mask, "W": np.ascontiguousarray(weight),
                "bias": bias}
    b, q, h, d, l, p = w.batch, w.queries, w.heads, w.head_dim, w.levels, w.points
    value = rng.standard_normal((b, w.spatial_size, h, d), dtype=np.float32)
    if w.location_model == "uniform":
        loc = rng.uniform(-0.05, 1.05, (b, q, h, l, p, 2)).astype(np.float32)
    elif w.location_model == "reference_gauss":
        ref = rng.uniform(0.0, 1.0, (b, q, 1, 1, 1, 2)).astype(np.float32)
        loc = ref + rng.standard_normal((b, q, h, l, p, 2), dtype=np.float32) * np.float32(w.sigma)
    elif w.location_model == "bev_grid":
        side = int(round(np.sqrt(q)))
        if side * side != q:
            raise ValidationError("bev_grid locations need a square query count")
        centre = (np.arange(side, dtype=np.float32) + np.float32(0.5)) / np.float32(side)
        gx, gy = np.meshgrid(centre, centre, indexing="xy")
        grid = np.stack([gx.reshape(-1), gy.reshape(-1)], axis=-1).reshape(1, q, 1, 1, 1, 2)
        loc = grid + rng.standard_normal((b, q, h, l, p, 2), dtype=np.float32) * np.float32(w.sigma)
    else:
        raise ValidationError(f"unknown location model {w.location_model!r}")
    logits = rng.standard_normal((b, q, h, l * p), dtype=np.float32)
    attn = _softmax_last(logits).reshape(b, q, h, l, p)
    return {"value": value, "sampling_locations": np.ascontiguousarray(loc, dtype=np.float32),
            "attention_weights": np.ascontiguousarray(attn)}


def build_msda_graph_for(w: MsdaWorkload, name: str | None = None) -> Graph:
    """One-node MSDeformableAttention graph with inferred output spec."""
    l, p = w.levels, w.points
    inputs = {
        "value": TensorSpec((w.batch, w.spatial_size, w.heads, w.head_dim), "float32"),
        "sampling_locations": TensorSpec((w.batch, w.queries, w.heads, l, p, 2), "float32"),
        "attention_weights": TensorSpec((w.batch, w.queries, w.heads, l, p), "float32"),
    }
    node = Node("msda", "MSDeformableAttention", ("value", "sampling_locations", "attention_weights"),
                ("output",), {"spatial_shapes": [list(s) for s in w.spatial_shapes]})
    g = Graph(name or f"bevformer_{w.name}_msda", inputs, ("output",), [node],
              metadata={"workload": w.name, "dtype": "float32"})
    g.value_specs.update(infer_node(node, g.value_specs))
    g.validate()
    return g


def build_dcn_graph_for(w: DcnWorkload, name: str | None = None, with_bias: bool = True) -> Graph:
    kh, kw = w.kernel
    ho, wo = w.out_hw
    k = kh * kw
    inputs = {
        "X": TensorSpec((w.batch, w.cin, w.height, w.width), "float32", "NCHW"),
        "offset": TensorSpec((w.batch, 2 * w.deform_groups * k, ho, wo), "float32", "NCHW"),
        "mask": TensorSpec((w.batch, w.deform_groups * k, ho, wo), "float32", "NCHW"),
        "W": TensorSpec((w.cout, w.cin // w.groups, kh, kw), "float32"),
    }
    names = ["X", "offset", "mask", "W"]
    if with_bias:
        inputs["bias"] = TensorSpec((w.cout,), "float32")
        names.append("bias")
    node = Node("dcn", "DeformConv2D", tuple(names), ("Y",), w.attrs())
    g = Graph(name or f"r101_{w.name}", inputs, ("Y",), [node], metadata={"workload": w.name})
    g.value_specs.update(infer_node(node, g.value_specs))
    g.validate()
    return g


# The reference's tiny profile: six cameras, C5 at 15x25, 2500 BEV queries,
# 8 heads of 32 channels, 8 points on one level (model.py:17-60).
_TINY_SLICE = MsdaWorkload("tiny_sca_slice", 6, 2500, 8, 32, 8, ((15, 25),), "uniform")


def build_msda_graph() -> Graph:
    """The FP32 BEVFormer-tiny spatial MSDA slice ``bevformer_tiny_msda`` (model.py:137-191)."""
    g = build_msda_graph_for(_TINY_SLICE, "bevformer_tiny_msda")
    g.metadata["reference_slice"] = {"name": "bevformer_tiny_spatial_cross_attention_msda",
                                     "kind": "fp32-reference-slice", "dtype": "float32"}
    return g


def make_msda_inputs(graph: Graph, seed: int = 7) -> dict:
    """Inputs for an MSDA graph drawn exactly like the reference's recipe (model.py:193-235):
    value ~ N(0,1), locations ~ U(-0.25,1.25), weights ~ U(0.01,1) normalised over (L,P)."""
    if isinstance(seed, bool) or not isinstance(seed, Integral):
        raise ValidationError("MSDA input seed must be an integer")
    names = ("value", "sampling_locations", "attention_weights")
    missing = [n for n in names if n not in graph.inputs]
    if missing:
        raise ValidationError(f"MSDA graph is missing inputs: {missing}")
    shp = {}
    for n in names:
        spec = graph.inputs[n]
        if not spec.is_static:
            raise ValidationError(f"MSDA input {n!r} must have a static shape")
        if spec.dtype != "float32":
            raise ValidationError(f"MSDA input {n!r} must have dtype float32")
        shp[n] = tuple(int(d) for d in spec.shape)
    rng = np.random.default_rng(int(seed))
    value = rng.normal(size=shp["value"]).astype(np.float32)
    loc = rng.uniform(-0.25, 1.25, size=shp["sampling_locations"]).astype(np.float32)
    attn = rng.uniform(np.float32(0.01), np.float32(1.0), size=shp["attention_weights"]).astype(np.float32)
    attn = attn / attn.sum(axis=(-2, -1), keepdims=True, dtype=np.float32)
    return {"value": np.ascontiguousarray(value, dtype=np.float32),
            "sampling_locations": np.ascontiguousarray(loc, dtype=np.float32),
            "attention_weights": np.ascontiguousarray(attn, dtype=np.float32)}


# --------------------------------------------------------------------------- #
# the sub-graphs BEVFormer builds around the sampling operators
# --------------------------------------------------------------------------- #

def build_sca_block_graph(samples: int, cameras: int, queries: int, heads: int, head_dim: int, spatial_shapes,
                          points_per_anchor: int, anchors: int, name: str = "bevformer_sca_block") -> Graph:
    """Spatial cross-attention from the projected tensors to the camera-averaged context, node for node as GAC
    builds it (src/gac/models/bevformer/spatial.py:160-188) minus the MatMul projections on either side:
    value view, offsets / normalizer + expanded reference, softmax over L*P, MSDeformableAttention, visibility
    multiply, camera sum, clamp-count divide.  ``fuse_deformable_sampling`` turns all of it into one launch."""
    n, q, h, d = samples * cameras, queries, heads, head_dim
    levels, points = len(spatial_shapes), points_per_anchor * anchors
    spatial = sum(int(a) * int(b) for a, b in spatial_shapes)
    c = h * d
    inputs = {
        "value_projected": TensorSpec((n, spatial, c), "float32"),
        "offset_flat": TensorSpec((n, q, h * levels * points * 2), "float32"),
        "reference_points": TensorSpec((samples, cameras, q, anchors, 2), "float32"),
        "attention_flat": TensorSpec((n, q, h * levels * points), "float32"),
        "visibility": TensorSpec((samples, cameras, q, 1), "float32"),
    }
    normalizer = np.asarray([[w, hh] for hh, w in spatial_shapes], np.float32).reshape(1, 1, 1, levels, 1, 1, 2)
    full = [n, q, h, levels, points_per_anchor, anchors, 2]
    nodes = [
        Node("value_heads", "Reshape", ("value_projected",), ("value_msda",), {"shape": [n, spatial, h, d]}),
        Node("offset_shape", "Reshape", ("offset_flat",), ("offsets",), {"shape": full}),
        Node("offset_normalize", "Div", ("offsets", "offset_normalizer"), ("normalized_offsets",)),
        Node("reference_flatten_cameras", "Reshape", ("reference_points",), ("reference_nqa2",), {"shape": [n, q, anchors, 2]}),
        Node("reference_axes", "Reshape", ("reference_nqa2",), ("reference_nq111a2",), {"shape": [n, q, 1, 1, 1, anchors, 2]}),
        Node("reference_expand", "Expand", ("reference_nq111a2",), ("reference_expanded",), {"shape": full}),
        Node("location_add", "Add", ("reference_expanded", "normalized_offsets"), ("locations_split",)),
        Node("location_shape", "Reshape", ("locations_split",), ("sampling_locations",), {"shape": [n, q, h, levels, points, 2]}),
        Node("attention_head_shape", "Reshape", ("attention_flat",), ("attention_by_head",), {"shape": [n, q, h, levels * points]}),
        Node("attention_softmax", "Softmax", ("attention_by_head",), ("attention_probability",), {"axis": -1}),
        Node("attention_shape", "Reshape", ("attention_probability",), ("attention_weights",), {"shape": [n, q, h, levels, points]}),
        Node("spatial_msda", "MSDeformableAttention", ("value_msda", "sampling_locations", "attention_weights"),
             ("camera_context",), {"spatial_shapes": [list(s) for s in spatial_shapes]}),
        Node("camera_context_shape", "Reshape", ("camera_context",), ("context_bcqc",), {"shape": [samples, cameras, q, c]}),
        Node("visibility_apply", "Mul", ("context_bcqc", "visibility"), ("masked_context",)),
        Node("camera_sum", "ReduceSum", ("masked_context",), ("context_sum",), {"axes": [1], "keepdims": False}),
        Node("visibility_sum", "ReduceSum", ("visibility",), ("visible_count",), {"axes": [1], "keepdims": False}),
        Node("visibility_clamp", "Clamp", ("visible_count",), ("safe_count",), {"min": 1.0}),
        Node("camera_average", "Div", ("context_sum", "safe_count"), ("averaged_context",)),
    ]
    g = Graph(name, inputs, ("averaged_context",), nodes, constants={"offset_normalizer": normalizer})
    g.validate()
    return g


def build_tsa_tail_graph(samples: int, queue: int, queries: int, heads: int, head_dim: int, bev_hw, points: int,
                         name: str = "bevformer_tsa_tail") -> Graph:
    """Temporal self-attention from the sampling operator to the queue mean (temporal.py:366-389)."""
    n = samples * queue
    c = heads * head_dim
    inputs = {
        "value_msda": TensorSpec((n, int(bev_hw[0]) * int(bev_hw[1]), heads, head_dim), "float32"),
        "sampling_locations": TensorSpec((n, queries, heads, 1, points, 2), "float32"),
        "attention_weights": TensorSpec((n, queries, heads, 1, points), "float32"),
    }
    nodes = [
        Node("temporal_msda", "MSDeformableAttention", ("value_msda", "sampling_locations", "attention_weights"),
             ("queue_context",), {"spatial_shapes": [[int(bev_hw[0]), int(bev_hw[1])]]}),
        Node("context_queue_shape", "Reshape", ("queue_context",), ("context_bqqc",), {"shape": [samples, queue, queries, c]}),
        Node("context_queue_mean", "ReduceMean", ("context_bqqc",), ("context",), {"axes": [1], "keepdims": False}),
    ]
    g = Graph(name, inputs, ("context",), nodes)
    g.validate()
    return g


def build_dcn_bottleneck_graph(w: DcnWorkload, constants: dict, three_way: bool = False, name: str | None = None) -> Graph:
    """The deformable 3x3 stage of an R101-DCN bottleneck as a model exporter writes it: a ``conv_offset`` convolution
    of ``3 * deform_groups * Kh * Kw`` channels over X, its output cut along the channels into offsets and mask
    scores (``three_way``: mmcv's ``chunk(3)`` with the first two pieces concatenated again), ``Sigmoid`` on the mask
    scores, ``DeformConv2D`` over the same X, ``BatchNorm``, ``ReLU``.  ``constants`` holds ``W_offset``, ``b_offset``,
    ``W``, ``bias`` and ``bn_scale`` / ``bn_bias`` / ``bn_mean`` / ``bn_variance``; X is the only input."""
    kh, kw = w.kernel
    k = kh * kw * w.deform_groups
    pads = [w.padding[0], w.padding[1], w.padding[0], w.padding[1]]
    conv = {"strides": list(w.stride), "pads": pads, "dilations": list(w.dilation)}

    def cut(begin, end):
        return {"starts": [begin], "ends": [end], "axes": [1], "steps": [1]}

    nodes = [Node("conv_offset", "Conv2D", ("X", "W_offset", "b_offset"), ("offset_mask",), conv)]
    if three_way:
        nodes += [Node("chunk_o1", "Slice", ("offset_mask",), ("o1",), cut(0, k)),
                  Node("chunk_o2", "Slice", ("offset_mask",), ("o2",), cut(k, 2 * k)),
                  Node("chunk_mask", "Slice", ("offset_mask",), ("mask_scores",), cut(2 * k, 3 * k)),
                  Node("offset_cat", "Concat", ("o1", "o2"), ("offset",), {"axis": 1})]
    else:
        nodes += [Node("take_offset", "Slice", ("offset_mask",), ("offset",), cut(0, 2 * k)),
                  Node("take_mask", "Slice", ("offset_mask",), ("mask_scores",), cut(2 * k, 3 * k))]
    nodes += [Node("mask_sigmoid", "Sigmoid", ("mask_scores",), ("mask",)),
              Node("conv2", "DeformConv2D", ("X", "offset", "mask", "W", "bias"), ("conv2_out",), w.attrs()),
              Node("bn2", "BatchNorm", ("conv2_out", "bn_scale", "bn_bias", "bn_mean", "bn_variance"), ("normed",),
                   {"epsilon": 1e-5}),
              Node("relu2", "ReLU", ("normed",), ("Y",))]
    g = Graph(name or f"r101_{w.name}_bottleneck", {"X": TensorSpec((w.batch, w.cin, w.height, w.width), "float32", "NCHW")},
              ("Y",), nodes, dict(constants))
    g.validate()
    return g


def build_dcn_block_graph(w: DcnWorkload, name: str | None = None) -> Graph:
    """``Sigmoid(mask scores) -> DeformConv2D -> BatchNorm -> ReLU`` as the R101-DCN bottleneck runs them as
    separate dispatches in GAC (175 Sigmoid dispatches in the base profile)."""
    kh, kw = w.kernel
    ho, wo = w.out_hw
    k = kh * kw
    inputs = {
        "X": TensorSpec((w.batch, w.cin, w.height, w.width), "float32", "NCHW"),
        "offset": TensorSpec((w.batch, 2 * w.deform_groups * k, ho, wo), "float32", "NCHW"),
        "mask_scores": TensorSpec((w.batch, w.deform_groups * k, ho, wo), "float32", "NCHW"),
        "W": TensorSpec((w.cout, w.cin // w.groups, kh, kw), "float32"),
        "bias": TensorSpec((w.cout,), "float32"),
        **{f"bn_{p}": TensorSpec((w.cout,), "float32") for p in ("scale", "bias", "mean", "variance")},
    }
    nodes = [
        Node("mask_sigmoid", "Sigmoid", ("mask_scores",), ("mask",)),
        Node("dcn", "DeformConv2D", ("X", "offset", "mask", "W", "bias"), ("conv2",), w.attrs()),
        Node("bn2", "BatchNorm", ("conv2", "bn_scale", "bn_bias", "bn_mean", "bn_variance"), ("normed",), {"epsilon": 1e-5}),
        Node("relu2", "ReLU", ("normed",), ("Y",)),
    ]
    g = Graph(name or f"r101_{w.name}_block", inputs, ("Y",), nodes)
    g.validate()
    return g
