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
THREADS_PER_CTA = 256

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


def msda_rows_per_cta(head_dim: int, samples: int, value_dtype: str = "float32") -> int | None:
    """Rows (batch, query, head) one CTA of the vector kernel covers; None = scalar fallback kernel.

    Mirrors the launch arithmetic of ``csrc/msda.cu``: CPL channels per lane
    (4 for float32, 8 for bfloat16), LPR = D / CPL lanes per row (a power of two
    up to 32), 256/LPR rows side by side, and up to 8 row batches per CTA while
    the CTA's tap table (samples padded to a multiple of 4) stays within 512 records.
    """
    cpl = 4 if value_dtype == "float32" else 8
    if head_dim % cpl:
        return None
    lpr = head_dim // cpl
    if lpr not in (1, 2, 4, 8, 16, 32):
        return None
    side = THREADS_PER_CTA // lpr
    cap = max(4, 512 // side)
    if samples <= cap:
        padded = -(-samples // 4) * 4
        return side * max(1, min(8, cap // padded))
    return side


def _plan(node: Node, specs: dict, options: dict) -> KernelLaunch:
    out_spec: TensorSpec = specs[node.outputs[0]]
    if node.op == FUSED_MSDA:
        b, q, h, l, p = node.attrs["dims"]
        value = specs[node.inputs[0]]
        storage = options.get("value_storage", "float32")
        rows = msda_rows_per_cta(value.shape[3], l * p, storage)
        grid = (math.ceil(b * q * h / rows), 1, 1) if rows else (math.ceil(b * q * h * value.shape[3] / THREADS_PER_CTA), 1, 1)
        what = [k for k in ("softmax",) if node.attrs.get(k)] + \
               (["coordinates"] if node.attrs.get("coordinates") == "offsets" else []) + \
               ([node.attrs["reduce"]] if node.attrs.get("reduce", "none") != "none" else [])
        candidates = (f"rows-vector-{storage}+" + "+".join(what),)
        return KernelLaunch(ENTRY_POINTS[node.op], node.id, node.inputs, node.outputs[0], grid,
                            (THREADS_PER_CTA, 1, 1), node.source_nodes, candidates)
    if node.op in ("DeformConv2D", "Conv2D"):
        n, cout, ho, wo = out_spec.shape
        grid = (math.ceil(n * ho * wo / 128), 1, 1)
        candidates = ("tcgen05-implicit-gemm-" + options.get("dcn_math", "f32x3"),)
    else:
        value, loc = specs[node.inputs[0]], specs[node.inputs[1]]
        b, q, h = loc.shape[0], loc.shape[1], loc.shape[2]
        samples = loc.shape[3] * loc.shape[4]
        if len(node.attrs["spatial_shapes"]) > MAX_LEVELS:
            _reject(node, f"at most {MAX_LEVELS} feature levels are supported")
        if loc.shape[4] > MAX_POINTS:
            _reject(node, f"at most {MAX_POINTS} sampling points per level are supported")
        storage = options.get("value_storage", "float32")
        rows = msda_rows_per_cta(value.shape[3], samples, storage)
        if rows is None:
            grid = (math.ceil(b * q * h * value.shape[3] / THREADS_PER_CTA), 1, 1)
            candidates = ("scalar-per-output",)
        else:
            grid = (math.ceil(b * q * h / rows), 1, 1)
            candidates = (f"rows-vector-{storage}",)
    return KernelLaunch(ENTRY_POINTS[node.op], node.id, node.inputs, node.outputs[0], grid,
                        (THREADS_PER_CTA, 1, 1), node.source_nodes, candidates)


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
