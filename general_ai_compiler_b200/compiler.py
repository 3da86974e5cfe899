"""Launch planning for the B200 backend, after ``src/gac/targets/cuda/compiler.py``.

``compile_cuda(graph)`` validates a graph of deformable-sampling ops and returns
a ``CudaProgram`` whose ``launches`` describe which ``libgacb.so`` entry point
runs each node (the reference returns generated CUDA-C plus ``KernelLaunch``
records, :40-80, :723-762).  No device is touched and nothing is generated: the
kernels are precompiled sm_100a code, so ``source`` names the entry points only.

Backend limits match the reference's checks: static positive dimensions,
C-contiguous float32 tensors below 2^31 elements (:201-222), at most 32 levels
and 64 points per level for MSDA (:179-185); non-float32 graphs raise
``BackendError`` (:145-148).
"""

from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field
from typing import Any

import numpy as np

from .errors import BackendError, ShapeInferenceError
from .ir import Graph, Node, TensorSpec
from .ops import FUSED_MSDA, MAX_LEVELS, MAX_POINTS, SUPPORTED_OPS, infer_node
from .passes import fuse_deformable_sampling, infer_neighbour_specs

TARGET = "cuda-sm100a"

ENTRY_POINTS = {
    "MSDeformableAttention": "gacb_msda_forward",
    "MSDeformableAttentionOffsets": "gacb_msda_offsets_forward",
    "DeformConv2D": "gacb_dcnv2_forward",
    "Conv2D": "gacb_conv2d_forward",
    FUSED_MSDA: "gacb_msda_run",
}
VIEW_OPS = ("Reshape",)      # no launch: the session aliases the input buffer


@dataclass(frozen=True)
class KernelLaunch:
    entry_point: str
    node_id: str
    inputs: tuple
    output: str
    grid: tuple
    block: tuple
    source_nodes: tuple
    implementation_candidates: tuple
    extra_outputs: tuple = ()      # a Conv2D whose channels go to two tensors: the second one


@dataclass
class CudaProgram:
    graph: Graph
    reference_graph: Graph
    source: str
    launches: tuple
    pass_reports: tuple = ()
    options: dict = field(default_factory=dict)

    def describe(self) -> dict[str, Any]:
        g = self.graph
        return {
            "schema_version": 1,
            "target": TARGET,
            "compute_capability": [10, 0],
            "artifact_kind": "precompiled-sm100a-library-with-launch-metadata",
            "device_code_compiled": True,
            "precision": "float32 accumulate; optional bfloat16 value storage (MSDA); "
                         "bf16 hi+lo pairs (three products, fp32-faithful) / TF32 / BF16 tensor-core products (DCNv2)",
            "name": g.name,
            "inputs": {k: s.to_dict() for k, s in g.inputs.items()},
            "outputs": {k: g.value_specs[k].to_dict() for k in g.outputs},
            "launches": [asdict(l) for l in self.launches],
            "pass_reports": list(self.pass_reports),
            "options": dict(self.options),
            "tensor_bytes_upper_bound": sum(s.nbytes for s in g.value_specs.values()),
        }


def _reject(node: Node, why: str):
    raise BackendError(f"{TARGET}: {node.op} node {node.id!r}: {why}")


def _check_specs(graph: Graph) -> None:
    for name, spec in graph.value_specs.items():
        if not spec.is_static or any(d <= 0 for d in spec.shape):
            raise BackendError(f"{TARGET}: {name!r} requires static, positive dimensions")
        if spec.dtype != "float32" or spec.layout not in ("contiguous", "NCHW"):
            raise BackendError(f"{TARGET}: {name!r} requires C-contiguous float32 storage, got {spec.dtype}/{spec.layout}")
        if math.prod(spec.shape) > 2**31 - 1:
            raise BackendError(f"{TARGET}: {name!r} exceeds the supported 32-bit indexing range")
    for name, value in graph.constants.items():
        if not np.all(np.isfinite(value)):
            raise BackendError(f"{TARGET}: constant {name!r} must contain finite values")


def _msda_launch(node: Node, value: TensorSpec, b: int, q: int, h: int, levels_points, shapes, storage: str):
    """(grid, block, kernel name, rows per thread block) of the MSDA launch, asked of the library itself
    (``gacb_msda_launch_geometry``): the kernels are precompiled, so only the library knows their shapes."""
    from . import native

    l, p = levels_points
    dtype = native.GACB_F32 if storage == "float32" else native.GACB_BF16
    geo = native.msda_launch_geometry(dtype, shapes, b, q, h, value.shape[3], p)
    return tuple(geo.grid), tuple(geo.block), geo.kernel.decode(), int(geo.units_per_cta)


def msda_rows_per_cta(head_dim: int, samples: int, value_dtype: str = "float32") -> int | None:
    """Rows (batch, query, head) one thread block of the vector kernel covers; None = one-thread-per-output kernel.
    Answered by the library for a one-level problem with ``samples`` points."""
    from . import native

    dtype = native.GACB_F32 if value_dtype == "float32" else native.GACB_BF16
    geo = native.msda_launch_geometry(dtype, [(1, 1)], 1, 4096, 1, head_dim, samples)
    return int(geo.units_per_cta) if geo.kernel.startswith(b"msda_rows") else None


def _plan(node: Node, specs: dict, options: dict) -> KernelLaunch:
    from . import native

    out_spec: TensorSpec = specs[node.outputs[0]]
    if node.op == FUSED_MSDA:
        b, q, h, l, p = node.attrs["dims"]
        value = specs[node.inputs[0]]
        storage = options.get("value_storage", "float32")
        grid, block, kernel, _ = _msda_launch(node, value, b, q, h, (l, p), node.attrs["spatial_shapes"], storage)
        what = [k for k in ("softmax",) if node.attrs.get(k)] + \
               (["coordinates"] if node.attrs.get("coordinates") == "offsets" else []) + \
               ([node.attrs["reduce"]] if node.attrs.get("reduce", "none") != "none" else [])
        # with a visibility operand the grid is an upper bound: thread blocks past the compacted row list return
        candidates = (kernel + ("+" + "+".join(what) if what else ""),)
        return KernelLaunch(ENTRY_POINTS[node.op], node.id, node.inputs, node.outputs[0], grid, block,
                            node.source_nodes, candidates)
    if node.op in ("DeformConv2D", "Conv2D"):
        x, w = specs[node.inputs[0]], specs[node.inputs[3 if node.op == "DeformConv2D" else 1]]
        math = native.DCN_MATH_MODES[options.get("dcn_math", "f32x3")]
        if node.op == "DeformConv2D":
            from .ops import dcn_attrs

            stride, padding, dilation, groups, dgroups = dcn_attrs(node)
            plain = False
        else:
            from .ops import conv_attrs

            stride, pads, dilation, groups = conv_attrs(node)
            padding, dgroups, plain = (pads[0], pads[1]), 1, True
        try:
            geo = native.dcnv2_launch_geometry(x.shape[0], x.shape[1], x.shape[2], x.shape[3], w.shape[0], w.shape[2],
                                               w.shape[3], stride, padding, dilation, groups, dgroups, math, plain=plain)
        except Exception as exc:
            _reject(node, str(exc))
        return KernelLaunch(ENTRY_POINTS[node.op], node.id, node.inputs, node.outputs[0], tuple(geo.grid),
                            tuple(geo.block), node.source_nodes, (geo.kernel.decode(),), tuple(node.outputs[1:]))
    value, loc = specs[node.inputs[0]], specs[node.inputs[1]]
    b, q, h = loc.shape[0], loc.shape[1], loc.shape[2]
    if len(node.attrs["spatial_shapes"]) > MAX_LEVELS:
        _reject(node, f"at most {MAX_LEVELS} feature levels are supported")
    if loc.shape[4] > MAX_POINTS:
        _reject(node, f"at most {MAX_POINTS} sampling points per level are supported")
    storage = options.get("value_storage", "float32")
    grid, block, kernel, _ = _msda_launch(node, value, b, q, h, (loc.shape[3], loc.shape[4]),
                                          node.attrs["spatial_shapes"], storage)
    return KernelLaunch(ENTRY_POINTS[node.op], node.id, node.inputs, node.outputs[0], grid, block,
                        node.source_nodes, (kernel,))


def compile_cuda(graph: Graph, *, fuse: bool = True, value_storage: str = "float32",
                 dcn_math: str = "f32x3") -> CudaProgram:
    """Validate semantics and plan launches.  No device access occurs.

    ``value_storage="bfloat16"`` makes sessions keep MSDA's ``value`` in bf16 on
    the device (float32 at the host boundary, float32 accumulation);
    ``dcn_math`` picks the DCNv2 tensor-core product ("f32x3", "tf32", "bf16").
    ``fuse=True`` first runs ``passes.fuse_deformable_sampling``: the softmax,
    coordinate arithmetic, visibility average / queue mean around an MSDA node
    and the sigmoid / BatchNorm / ReLU around a convolution become part of that
    node's launch; with ``fuse=False`` a graph may only hold the bare operators.
    ``Reshape`` nodes that remain are views (no launch).
    """
    if value_storage not in ("float32", "bfloat16"):
        raise BackendError(f"{TARGET}: value_storage must be 'float32' or 'bfloat16'")
    if dcn_math not in ("f32x3", "tf32", "bf16"):
        raise BackendError(f"{TARGET}: dcn_math must be 'f32x3', 'tf32' or 'bf16'")
    work = graph.clone()
    work.validate()
    reference_graph = work.clone()
    reports = []
    if fuse:
        work, fusion_report = fuse_deformable_sampling(work)
        reports.append(fusion_report)
    for node in work.nodes:
        if node.op not in SUPPORTED_OPS and node.op != FUSED_MSDA and node.op not in VIEW_OPS:
            raise BackendError(f"{TARGET}: op {node.op!r} (node {node.id!r}) is outside the deformable-sampling path")
    infer_neighbour_specs(work)
    for node in work.nodes:
        missing = [o for o in node.outputs if o not in work.value_specs]
        if missing:
            raise ShapeInferenceError(f"node {node.id!r}: cannot infer the shape of {missing[0]!r}")
        if node.op in VIEW_OPS:
            src, dst = work.value_specs[node.inputs[0]], work.value_specs[node.outputs[0]]
            if src.numel != dst.numel:
                raise ShapeInferenceError(f"Reshape node {node.id!r} changes the element count")
    _check_specs(work)
    options = {"value_storage": value_storage, "dcn_math": dcn_math}
    launches = tuple(_plan(node, work.value_specs, options) for node in work.nodes if node.op not in VIEW_OPS)
    source = "\n".join(f"// {l.node_id}: {l.entry_point} grid={l.grid} block={l.block}" for l in launches)
    reports.append({"name": "shape-inference", "changed": True, "details": {"nodes": len(work.nodes), "fuse": bool(fuse)}})
    return CudaProgram(work, reference_graph, source, launches, tuple(reports), options)
