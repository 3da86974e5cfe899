"""Operator registry for the deformable-sampling path.

Mirrors the op API of the reference (``src/gac/core/ops.py``): ``infer_node``
(:440-442) derives output specs, ``evaluate_op`` (:854-858) executes one op on
NumPy arrays.  Here ``evaluate_op`` runs on the B200 through ``libgacb.so`` --
host arrays in, host arrays out -- and raises when no device or library is
available; it never computes on the CPU.

Device-resident entry points (``msda_forward``, ``msda_offsets_forward``,
``dcnv2_forward``) take CUDA ``torch.Tensor`` objects: torch is used for device
memory and streams only, the arithmetic is in the hand-written kernels.

Supported ops and their contracts:

``MSDeformableAttention``         inputs (value [B,S,H,D], sampling_locations
    [B,Q,H,L,P,2], attention_weights [B,Q,H,L,P]); attr ``spatial_shapes``
    [[H_l, W_l], ...]; output [B,Q,H*D].  Contract of ops.py:387-437.
    Optional attr ``softmax: true`` (both MSDA ops): the third input holds raw
    scores and the Softmax node that precedes the op in the BEVFormer graphs
    (models/bevformer/spatial.py:172-174) is folded into the kernel.
``MSDeformableAttentionOffsets``  the fused-coordinate form
    gac.ms_deform_attn_offsets: inputs (value, offsets, attention_weights,
    normalizer, reference); attrs ``spatial_shapes``, ``coordinate_shape``,
    ``reference_first``.  Contract of native/lib/Dialect.cpp:398-447.
``DeformConv2D``                  gac.deform_conv2d / MMCVModulatedDeformConv2d:
    inputs (X, offset, mask, W[, bias]); attrs ``stride``, ``padding``,
    ``dilation`` (pairs), ``groups``, ``deform_groups``.  Contract of
    native/lib/Dialect.cpp:272-360.
``Conv2D``                        the plain convolutions next to DCNv2 (above all
    ``conv_offset``): inputs (X, W[, bias]); attrs ``strides``, ``dilations``
    (pairs), ``pads`` (top, left, bottom, right), ``groups``; ``relu`` folds the
    reference's conv2d_relu.  Contract of src/gac/core/ops.py:615-645.
"""

from __future__ import annotations

import ctypes
from typing import Any, Mapping, Sequence

import numpy as np

from . import native
from .errors import BackendError, DeviceUnavailableError, EvaluationError, ShapeInferenceError
from .ir import Node, TensorSpec

SUPPORTED_OPS = frozenset({"MSDeformableAttention", "MSDeformableAttentionOffsets", "DeformConv2D", "Conv2D"})

MAX_LEVELS = 32
MAX_POINTS = 64


# --------------------------------------------------------------------------- #
# shape inference
# --------------------------------------------------------------------------- #

def _is_int(v: object) -> bool:
    return isinstance(v, (int, np.integer)) and not isinstance(v, bool)


def _same(left, right) -> bool:
    """Two dimensions agree when equal, or when either is not a static int."""
    return not (isinstance(left, int) and isinstance(right, int)) or left == right


def spatial_shapes_of(attrs: Mapping[str, Any], err=ShapeInferenceError, who: str = "MSDeformableAttention"):
    raw = attrs.get("spatial_shapes")
    if not isinstance(raw, (list, tuple, np.ndarray)) or len(raw) == 0:
        raise err(f"{who} requires non-empty spatial_shapes")
    pairs = []
    for k, pair in enumerate(raw):
        if not isinstance(pair, (list, tuple, np.ndarray)) or len(pair) != 2:
            raise err(f"{who} spatial_shapes[{k}] must be [height, width]")
        h, w = pair
        if not _is_int(h) or not _is_int(w) or int(h) <= 0 or int(w) <= 0:
            raise err(f"{who} spatial shapes must contain positive integers")
        pairs.append((int(h), int(w)))
    return tuple(pairs)


def _floating(node: Node, spec: TensorSpec) -> None:
    if not np.issubdtype(np.dtype(spec.dtype), np.floating):
        raise ShapeInferenceError(f"{node.op} node {node.id!r} requires floating point input, got {spec.dtype}")


def _infer_msda(node: Node, specs: Sequence[TensorSpec], fused: bool) -> TensorSpec:
    want = 5 if fused else 3
    if len(specs) != want:
        raise ShapeInferenceError(f"{node.op} node {node.id!r} expects {want} inputs, got {len(specs)}")
    value, loc, attn = specs[0], specs[1], specs[2]
    for s in specs:
        _floating(node, s)
    if len({s.dtype for s in specs}) != 1:
        raise ShapeInferenceError(f"{node.op} node {node.id!r} requires all inputs to have one dtype")
    if (value.rank, loc.rank, attn.rank) != (4, 6, 5):
        raise ShapeInferenceError(
            f"{node.op} node {node.id!r} expects ranks [4, 6, 5], got [{value.rank}, {loc.rank}, {attn.rank}]")
    if loc.shape[-1] != 2:
        raise ShapeInferenceError(f"{node.op} node {node.id!r} sampling_locations last dimension must be 2")
    shapes = spatial_shapes_of(node.attrs, who=f"{node.op} node {node.id!r}")
    if loc.shape[3] != len(shapes) or attn.shape[3] != len(shapes):
        raise ShapeInferenceError(
            f"{node.op} node {node.id!r} level dimension must equal len(spatial_shapes)={len(shapes)}")
    total = sum(h * w for h, w in shapes)
    if isinstance(value.shape[1], int) and value.shape[1] != total:
        raise ShapeInferenceError(
            f"{node.op} node {node.id!r} value spatial dimension {value.shape[1]} does not equal sum(H*W)={total}")
    for left, right, what in (
        (value.shape[0], loc.shape[0], "batch"), (value.shape[0], attn.shape[0], "batch"),
        (loc.shape[1], attn.shape[1], "query"), (value.shape[2], loc.shape[2], "head"),
        (value.shape[2], attn.shape[2], "head"), (loc.shape[4], attn.shape[4], "point"),
    ):
        if not _same(left, right):
            raise ShapeInferenceError(f"{node.op} {what} dimensions do not match: {left!r} versus {right!r}")
    if fused:
        norm, ref = specs[3], specs[4]
        coord = node.attrs.get("coordinate_shape")
        if not isinstance(coord, (list, tuple)) or not coord or not all(_is_int(c) and int(c) > 0 for c in coord):
            raise ShapeInferenceError(f"{node.op} node {node.id!r} requires a positive coordinate_shape")
        if loc.is_static and int(np.prod(coord, dtype=np.int64)) != loc.numel:
            raise ShapeInferenceError(f"{node.op} node {node.id!r} coordinate_shape does not cover the locations")
        if norm.rank > 6 or ref.rank > len(coord):
            raise ShapeInferenceError(f"{node.op} node {node.id!r} normalizer/reference rank is too large")
        for have, full, what in ((norm.shape, loc.shape, "normalizer"), (ref.shape, tuple(coord), "reference")):
            padded = (1,) * (len(full) - len(have)) + tuple(have)
            if any(h != 1 and not _same(h, f) for h, f in zip(padded, full)):
                raise ShapeInferenceError(f"{node.op} node {node.id!r} {what} {have} does not broadcast to {full}")
    heads, hdim = value.shape[2], value.shape[3]
    channels = heads * hdim if isinstance(heads, int) and isinstance(hdim, int) else None
    return TensorSpec((value.shape[0], loc.shape[1], channels), value.dtype)


def _pair(node: Node, key: str, default: int, minimum: int):
    raw = node.attrs.get(key, [default, default])
    if _is_int(raw):
        raw = [raw, raw]
    if not isinstance(raw, (list, tuple)) or len(raw) != 2 or not all(_is_int(v) for v in raw):
        raise ShapeInferenceError(f"DeformConv2D node {node.id!r} attribute {key!r} must be a pair of integers")
    if any(int(v) < minimum for v in raw):
        raise ShapeInferenceError(
            f"DeformConv2D node {node.id!r} requires positive stride/dilation/groups and nonnegative padding")
    return int(raw[0]), int(raw[1])


def dcn_attrs(node: Node):
    """(stride, padding, dilation, groups, deform_groups) with the reference's defaults."""
    stride = _pair(node, "stride", 1, 1)
    padding = _pair(node, "padding", 0, 0)
    dilation = _pair(node, "dilation", 1, 1)
    groups = node.attrs.get("groups", 1)
    dgroups = node.attrs.get("deform_groups", 1)
    if not _is_int(groups) or not _is_int(dgroups) or int(groups) <= 0 or int(dgroups) <= 0:
        raise ShapeInferenceError(
            f"DeformConv2D node {node.id!r} requires positive stride/dilation/groups and nonnegative padding")
    return stride, padding, dilation, int(groups), int(dgroups)


def _infer_dcn(node: Node, specs: Sequence[TensorSpec]) -> TensorSpec:
    if node.attrs.get("batch_norm"):
        # folded inference BatchNorm: (X, offset, mask, W, bias, scale, bn_bias, mean, variance)
        if len(specs) != 9 or any(tuple(s.shape) != (specs[3].shape[0],) for s in specs[5:]):
            raise ShapeInferenceError(f"DeformConv2D node {node.id!r} with batch_norm needs nine inputs, the last "
                                      "four of shape [C]")
        specs = specs[:5]
    if len(specs) not in (4, 5):
        raise ShapeInferenceError(f"DeformConv2D node {node.id!r} expects 4 or 5 inputs, got {len(specs)}")
    if any(s.dtype != "float32" for s in specs):
        raise ShapeInferenceError("DeformConv2D currently requires FP32 tensors")
    stride, padding, dilation, groups, dgroups = dcn_attrs(node)
    x, offset, mask, weight = specs[:4]
    if any(s.rank != 4 for s in (x, offset, mask, weight)):
        raise ShapeInferenceError("DeformConv2D expects X/offset/mask NCHW and W OIHW rank-four tensors")
    if len(specs) == 5 and specs[4].rank != 1:
        raise ShapeInferenceError("DeformConv2D bias must be [output_channels]")
    cin, cout = x.shape[1], weight.shape[0]
    if (isinstance(cin, int) and (cin <= 0 or cin % groups or cin % dgroups)) or (
            isinstance(cout, int) and (cout <= 0 or cout % groups)):
        raise ShapeInferenceError("DeformConv2D channels must be positive and divisible by their groups")
    if isinstance(weight.shape[1], int) and isinstance(cin, int) and weight.shape[1] * groups != cin:
        raise ShapeInferenceError("DeformConv2D input channels disagree with grouped weights")
    if len(specs) == 5 and not _same(specs[4].shape[0], cout):
        raise ShapeInferenceError("DeformConv2D bias must be [output_channels]")
    out = [x.shape[0], cout, None, None]
    for d in range(2):
        k, size = weight.shape[2 + d], x.shape[2 + d]
        if isinstance(k, int) and k <= 0:
            raise ShapeInferenceError("DeformConv2D kernel extents must be positive")
        if not isinstance(k, int) or not isinstance(size, int):
            continue
        padded, span = size + 2 * padding[d], dilation[d] * (k - 1) + 1
        if padded < span:
            raise ShapeInferenceError("DeformConv2D kernel exceeds padded input")
        out[2 + d] = (padded - span) // stride[d] + 1
    if isinstance(weight.shape[2], int) and isinstance(weight.shape[3], int):
        points = weight.shape[2] * weight.shape[3] * dgroups
        for spec, channels in ((offset, 2 * points), (mask, points)):
            if not _same(spec.shape[1], channels):
                raise ShapeInferenceError(
                    "DeformConv2D offset/mask channels must be 2*deform_groups*kH*kW / deform_groups*kH*kW")
            for d in (0, 2, 3):
                if not _same(spec.shape[d], out[d]):
                    raise ShapeInferenceError("DeformConv2D offset/mask batch or spatial dimensions disagree")
    return TensorSpec(tuple(out), x.dtype, x.layout)


def conv_attrs(node: Node):
    """(strides, pads(top, left, bottom, right), dilations, groups) of a Conv2D node with the reference's defaults
    and checks (src/gac/core/ops.py:626-642)."""
    def ints(key, length, default, minimum):
        raw = node.attrs.get(key, default)
        if not isinstance(raw, (list, tuple)) or len(raw) != length or not all(_is_int(v) for v in raw):
            raise ShapeInferenceError(f"Conv2D node {node.id!r} attribute {key!r} must be {length} integers")
        if any(int(v) < minimum for v in raw):
            raise ShapeInferenceError(f"Conv2D node {node.id!r} attribute {key!r} must be >= {minimum}")
        return tuple(int(v) for v in raw)

    groups = node.attrs.get("groups", 1)
    if not _is_int(groups) or int(groups) <= 0:
        raise ShapeInferenceError(f"Conv2D node {node.id!r} groups must be positive")
    return ints("strides", 2, (1, 1), 1), ints("pads", 4, (0, 0, 0, 0), 0), ints("dilations", 2, (1, 1), 1), int(groups)


def conv_output_hw(H, W, Kh, Kw, strides, pads, dilations):
    return ((H + pads[0] + pads[2] - dilations[0] * (Kh - 1) - 1) // strides[0] + 1,
            (W + pads[1] + pads[3] - dilations[1] * (Kw - 1) - 1) // strides[1] + 1)


def _infer_conv(node: Node, specs: Sequence[TensorSpec]) -> TensorSpec:
    if len(specs) not in (2, 3):
        raise ShapeInferenceError(f"Conv2D node {node.id!r} expects 2 or 3 inputs, got {len(specs)}")
    if any(s.dtype != "float32" for s in specs):
        raise ShapeInferenceError("Conv2D requires FP32 tensors on this backend")
    x, weight = specs[:2]
    if x.rank != 4 or weight.rank != 4:
        raise ShapeInferenceError(f"Conv2D node {node.id!r} expects NCHW input and OIHW weight")
    strides, pads, dilations, groups = conv_attrs(node)
    cin, cout = x.shape[1], weight.shape[0]
    if isinstance(cin, int) and cin % groups:
        raise ShapeInferenceError(f"Conv2D node {node.id!r} input channels are not divisible by groups")
    if isinstance(cout, int) and cout % groups:
        raise ShapeInferenceError(f"Conv2D node {node.id!r} output channels are not divisible by groups")
    if isinstance(cin, int) and isinstance(weight.shape[1], int) and weight.shape[1] * groups != cin:
        raise ShapeInferenceError(f"Conv2D node {node.id!r} weight channels do not match groups")
    if len(specs) == 3 and tuple(specs[2].shape) != (cout,):
        raise ShapeInferenceError(f"Conv2D node {node.id!r} bias must have shape [out_channels]")
    out = [x.shape[0], cout, None, None]
    if all(isinstance(v, int) for v in (x.shape[2], x.shape[3], weight.shape[2], weight.shape[3])):
        ho, wo = conv_output_hw(x.shape[2], x.shape[3], weight.shape[2], weight.shape[3], strides, pads, dilations)
        if ho <= 0 or wo <= 0:
            raise ShapeInferenceError("convolution or pooling produces a non-positive dimension")
        out[2], out[3] = ho, wo
    return TensorSpec(tuple(out), x.dtype, x.layout)


FUSED_MSDA = "MSDeformableAttentionFused"     # produced by passes.fuse_deformable_sampling only


def _infer_msda_fused(node: Node, specs: Sequence[TensorSpec]) -> TensorSpec:
    """MSDA with its neighbours folded in: operands are named by attr ``operands``; tensors may arrive in any
    view of the right element count (the launch re-views them), so only counts are checked here."""
    a = node.attrs
    names = list(a.get("operands", ()))
    if len(names) != len(specs) or names[:3] != ["value", "locations", "attention"]:
        raise ShapeInferenceError(f"{node.op} node {node.id!r} has a malformed operand list")
    by = dict(zip(names, specs))
    try:
        B, Q, H, L, P = (int(v) for v in a["dims"])
    except (KeyError, TypeError, ValueError) as exc:
        raise ShapeInferenceError(f"{node.op} node {node.id!r} needs dims [B,Q,H,L,P]") from exc
    value = by["value"]
    if value.rank != 4 or any(s.dtype != "float32" for s in specs):
        raise ShapeInferenceError(f"{node.op} node {node.id!r} needs a rank-4 float32 value tensor")
    shapes = spatial_shapes_of(a, ShapeInferenceError)
    if len(shapes) != L or value.shape[0] != B or value.shape[2] != H or value.shape[1] != sum(h * w for h, w in shapes):
        raise ShapeInferenceError(f"{node.op} node {node.id!r}: value does not match dims / spatial_shapes")
    want = {"locations": B * Q * H * L * P * 2, "attention": B * Q * H * L * P, "visibility": B * Q}
    for key, count in want.items():
        if key in by and by[key].is_static and by[key].numel != count:
            raise ShapeInferenceError(f"{node.op} node {node.id!r}: {key} must hold {count} elements")
    group = int(a.get("group", 1))
    if a.get("reduce", "none") not in REDUCE_MODES or group < 1 or B % group:
        raise ShapeInferenceError(f"{node.op} node {node.id!r}: bad reduce/group")
    if a.get("reduce") == "masked_average" and "visibility" not in by:
        raise ShapeInferenceError(f"{node.op} node {node.id!r}: the masked average needs a visibility operand")
    if (a.get("coordinates") == "offsets") != ("normalizer" in by and "reference" in by):
        raise ShapeInferenceError(f"{node.op} node {node.id!r}: fused coordinates need normalizer and reference")
    lead = B // group if a.get("reduce", "none") != "none" else B
    return TensorSpec((lead, Q, H * value.shape[3]), "float32")


def infer_node(node: Node, value_specs: Mapping[str, TensorSpec]) -> dict:
    """Output specs of ``node`` from the specs of its inputs."""
    if node.op not in SUPPORTED_OPS and node.op != FUSED_MSDA:
        raise ShapeInferenceError(f"unsupported op {node.op!r} in node {node.id!r}")
    try:
        specs = [value_specs[name] for name in node.inputs]
    except KeyError as exc:
        raise ShapeInferenceError(f"node {node.id!r} uses unknown value {exc.args[0]!r}") from exc
    if node.op == "Conv2D" and node.attrs.get("split_at") is not None:
        # produced by passes.fuse_deformable_sampling: the output channels go to two tensors, [0, c) and [c, Cout)
        whole = _infer_conv(node, specs)
        cut = node.attrs["split_at"]
        if len(node.outputs) != 2 or not _is_int(cut) or not isinstance(whole.shape[1], int) or not 0 < int(cut) < whole.shape[1]:
            raise ShapeInferenceError(f"Conv2D node {node.id!r}: split_at needs two outputs and a cut inside the channels")
        lo = (whole.shape[0], int(cut), *whole.shape[2:])
        hi = (whole.shape[0], whole.shape[1] - int(cut), *whole.shape[2:])
        return {node.outputs[0]: TensorSpec(lo, whole.dtype, whole.layout), node.outputs[1]: TensorSpec(hi, whole.dtype, whole.layout)}
    if len(node.outputs) != 1:
        raise ShapeInferenceError(f"{node.op} node {node.id!r} must have exactly one output")
    if node.op == FUSED_MSDA:
        spec = _infer_msda_fused(node, specs)
    elif node.op == "DeformConv2D":
        spec = _infer_dcn(node, specs)
    elif node.op == "Conv2D":
        spec = _infer_conv(node, specs)
    else:
        spec = _infer_msda(node, specs, fused=node.op == "MSDeformableAttentionOffsets")
    return {node.outputs[0]: spec}


# --------------------------------------------------------------------------- #
# device-resident entry points (torch CUDA tensors in, torch CUDA tensor out)
# --------------------------------------------------------------------------- #

def _torch():
    import torch

    return torch


def require_device(device_id: int = 0):
    """Fail loudly unless an sm_100 device and the native library are usable."""
    torch = _torch()
    lib = native.load()
    if not torch.cuda.is_available():
        raise DeviceUnavailableError("no CUDA device is visible; there is no CPU fallback")
    n = lib.gacb_device_count()
    if n <= 0 or not 0 <= device_id < n:
        raise DeviceUnavailableError(f"CUDA device {device_id} does not exist (device count: {n})")
    cap = lib.gacb_device_capability(device_id)
    if cap // 10 != 10:
        raise DeviceUnavailableError(
            f"device {device_id} has compute capability {cap // 10}.{cap % 10}; this library holds sm_100a code only")
    return torch.device("cuda", device_id)


def _check_tensor(t, name: str, dtype, device=None):
    torch = _torch()
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise EvaluationError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise EvaluationError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise EvaluationError(f"{name} must be C-contiguous")
    if device is not None and t.device != device:
        raise EvaluationError(f"{name} lives on {t.device}, expected {device}")
    if t.data_ptr() % 16:
        raise EvaluationError(f"{name} must be 16-byte aligned")


def _stream_ptr(stream) -> int:
    torch = _torch()
    s = stream if stream is not None else torch.cuda.current_stream()
    return int(s.cuda_stream)


def _msda_dims(value, loc, attn, shapes):
    if value.dim() != 4 or loc.dim() != 6 or attn.dim() != 5:
        raise EvaluationError("MSDeformableAttention expects value/location/weight ranks [4, 6, 5]")
    B, S, H, D = value.shape
    if loc.shape[-1] != 2:
        raise EvaluationError("MSDeformableAttention locations last dimension must be 2")
    Q, L, P = loc.shape[1], loc.shape[3], loc.shape[4]
    if (loc.shape[0] != B or attn.shape[0] != B or attn.shape[1] != Q or loc.shape[2] != H
            or attn.shape[2] != H or L != len(shapes) or attn.shape[3] != L or attn.shape[4] != P
            or S != sum(h * w for h, w in shapes)):
        raise EvaluationError("MSDeformableAttention input shapes are inconsistent")
    return B, S, H, D, Q, L, P


def msda_forward(value, locations, weights, spatial_shapes, *, out=None, q_range=None, stream=None,
                 softmax=False):
    """MSDA on device tensors.  ``value`` is float32 or bfloat16 (storage only);
    locations/weights float32; returns float32 ``[B,Q,H*D]``.  ``q_range`` =
    (q_begin, q_end) limits the queries that are computed.  ``softmax=True``:
    ``weights`` holds raw scores and the softmax over each row's L*P scores is
    formed inside the kernel."""
    torch = _torch()
    lib = native.load()
    shapes = spatial_shapes_of({"spatial_shapes": spatial_shapes}, EvaluationError)
    if value.dtype not in (torch.float32, torch.bfloat16):
        raise EvaluationError("MSDeformableAttention value must be float32 or bfloat16 on this backend")
    _check_tensor(value, "value", value.dtype)
    _check_tensor(locations, "sampling_locations", torch.float32, value.device)
    _check_tensor(weights, "attention_weights", torch.float32, value.device)
    B, S, H, D, Q, L, P = _msda_dims(value, locations, weights, shapes)
    if out is None:
        out = torch.empty((B, Q, H * D), dtype=torch.float32, device=value.device)
    else:
        _check_tensor(out, "out", torch.float32, value.device)
        if tuple(out.shape) != (B, Q, H * D):
            raise EvaluationError(f"out must have shape {(B, Q, H * D)}")
    q0, q1 = (0, Q) if q_range is None else (int(q_range[0]), int(q_range[1]))
    table = native.int32_table(v for pair in shapes for v in pair)
    dt = native.GACB_F32 if value.dtype == torch.float32 else native.GACB_BF16
    with torch.cuda.device(value.device):
        entry = lib.gacb_msda_logits_forward if softmax else lib.gacb_msda_forward
        rc = entry(value.data_ptr(), dt, locations.data_ptr(), weights.data_ptr(), out.data_ptr(),
                   table, L, B, S, Q, H, D, P, q0, q1, _stream_ptr(stream))
    native.check(rc, "gacb_msda_logits_forward" if softmax else "gacb_msda_forward")
    return out


def _bcast_shape(have, full, what):
    padded = (1,) * (len(full) - len(have)) + tuple(int(v) for v in have)
    if len(padded) != len(full) or any(h != 1 and h != f for h, f in zip(padded, full)):
        raise EvaluationError(f"{what} shape {tuple(have)} does not broadcast to {tuple(full)}")
    return padded


def msda_offsets_forward(value, offsets, weights, normalizer, reference, spatial_shapes, coordinate_shape,
                         reference_first=False, *, out=None, q_range=None, stream=None, softmax=False):
    """Fused-coordinate MSDA: locations = offsets / normalizer (+) reference, formed in the kernel
    (and, with ``softmax=True``, the attention softmax over raw scores as well)."""
    torch = _torch()
    lib = native.load()
    shapes = spatial_shapes_of({"spatial_shapes": spatial_shapes}, EvaluationError)
    if value.dtype not in (torch.float32, torch.bfloat16):
        raise EvaluationError("MSDeformableAttention value must be float32 or bfloat16 on this backend")
    _check_tensor(value, "value", value.dtype)
    for t, name in ((offsets, "offsets"), (weights, "attention_weights"), (normalizer, "normalizer"),
                    (reference, "reference")):
        _check_tensor(t, name, torch.float32, value.device)
    B, S, H, D, Q, L, P = _msda_dims(value, offsets, weights, shapes)
    coord = tuple(int(c) for c in coordinate_shape)
    if not 1 <= len(coord) <= 8 or int(np.prod(coord, dtype=np.int64)) != offsets.numel():
        raise EvaluationError("coordinate_shape must have rank 1..8 and cover the locations")
    nshape = _bcast_shape(normalizer.shape, (B, Q, H, L, P, 2), "normalizer")
    rshape = _bcast_shape(reference.shape, coord, "reference")
    if out is None:
        out = torch.empty((B, Q, H * D), dtype=torch.float32, device=value.device)
    q0, q1 = (0, Q) if q_range is None else (int(q_range[0]), int(q_range[1]))
    dt = native.GACB_F32 if value.dtype == torch.float32 else native.GACB_BF16
    with torch.cuda.device(value.device):
        entry = lib.gacb_msda_offsets_logits_forward if softmax else lib.gacb_msda_offsets_forward
        rc = entry(
            value.data_ptr(), dt, offsets.data_ptr(), weights.data_ptr(), normalizer.data_ptr(),
            reference.data_ptr(), out.data_ptr(), native.int32_table(v for pair in shapes for v in pair),
            L, B, S, Q, H, D, P, native.int32_table(nshape), native.int32_table(coord),
            native.int32_table(rshape), len(coord), 1 if reference_first else 0, q0, q1, _stream_ptr(stream))
    native.check(rc, "gacb_msda_offsets_forward")
    return out


REDUCE_MODES = {"none": 0, "masked_average": 1, "mean": 2}


def msda_group_forward(value, locations, attention, spatial_shapes, *, group=1, reduce="none", visibility=None,
                       softmax=False, normalizer=None, reference=None, coordinate_shape=None, reference_first=False,
                       scratch=None, out=None, q_range=None, stream=None, compact=None):
    """MSDA followed by the reduction BEVFormer applies over groups of batch entries (``gacb_msda_run``).

    ``reduce="masked_average"`` (spatial cross-attention, spatial.py:183-188): batch entries are ``group`` cameras
    per sample, ``visibility`` is ``[B,Q]`` or ``[b,cam,Q,1]`` of 0/1; invisible (camera, query) rows are never
    sampled and the result is ``sum_cam vis*ctx / max(sum_cam vis, 1)`` of shape ``[B/group, Q, H*D]``.
    ``reduce="mean"`` (temporal self-attention, temporal.py:374-389): plain mean over the group.
    ``reduce="none"`` with ``visibility``: per-entry output ``[B,Q,H*D]`` whose masked rows are left untouched.
    ``scratch`` is the per-entry ``[B,Q,H*D]`` buffer the reduction reads (allocated here when omitted).
    ``compact`` is an optional int32 device buffer of ``B*Q + 4`` elements: the visible rows are then compacted
    first and the gather kernel runs dense CTAs over them."""
    torch = _torch()
    lib = native.load()
    if reduce not in REDUCE_MODES:
        raise EvaluationError(f"reduce must be one of {sorted(REDUCE_MODES)}")
    shapes = spatial_shapes_of({"spatial_shapes": spatial_shapes}, EvaluationError)
    if value.dtype not in (torch.float32, torch.bfloat16):
        raise EvaluationError("MSDeformableAttention value must be float32 or bfloat16 on this backend")
    _check_tensor(value, "value", value.dtype)
    _check_tensor(locations, "sampling_locations", torch.float32, value.device)
    _check_tensor(attention, "attention_weights", torch.float32, value.device)
    B, S, H, D, Q, L, P = _msda_dims(value, locations, attention, shapes)
    group = int(group)
    if group < 1 or B % group:
        raise EvaluationError(f"batch {B} is not a multiple of group {group}")
    desc = native.MsdaDesc()
    keep = []       # keeps ctypes tables alive until the call returns
    if visibility is not None:
        _check_tensor(visibility, "visibility", torch.float32, value.device)
        if visibility.numel() != B * Q:
            raise EvaluationError(f"visibility must have {B * Q} elements ([B,Q]), got {visibility.numel()}")
        desc.visibility = visibility.data_ptr()
    elif reduce == "masked_average":
        raise EvaluationError("the masked average needs a visibility tensor")
    if reduce == "mean" and visibility is not None:
        # masked rows are never written by the gather kernel, and the plain mean reads every row
        raise EvaluationError('reduce="mean" cannot be combined with visibility; use reduce="masked_average"')
    if (normalizer is None) != (reference is None):
        raise EvaluationError("normalizer and reference come together")
    if normalizer is not None:
        _check_tensor(normalizer, "normalizer", torch.float32, value.device)
        _check_tensor(reference, "reference", torch.float32, value.device)
        coord = tuple(int(c) for c in (coordinate_shape or locations.shape))
        if not 1 <= len(coord) <= 8 or int(np.prod(coord, dtype=np.int64)) != locations.numel():
            raise EvaluationError("coordinate_shape must have rank 1..8 and cover the locations")
        tables = [native.int32_table(_bcast_shape(normalizer.shape, (B, Q, H, L, P, 2), "normalizer")),
                  native.int32_table(coord), native.int32_table(_bcast_shape(reference.shape, coord, "reference"))]
        keep += tables
        desc.normalizer, desc.reference = normalizer.data_ptr(), reference.data_ptr()
        desc.norm_shape, desc.coord_shape, desc.ref_shape = tables
        desc.coord_rank, desc.reference_first = len(coord), 1 if reference_first else 0
    per_entry = (B, Q, H * D)
    if reduce == "none":
        if out is None:
            out = torch.zeros(per_entry, dtype=torch.float32, device=value.device)
        ctx, result = out, out
    else:
        ctx = scratch if scratch is not None else torch.empty(per_entry, dtype=torch.float32, device=value.device)
        if out is None:
            out = torch.empty((B // group, Q, H * D), dtype=torch.float32, device=value.device)
        _check_tensor(out, "out", torch.float32, value.device)
        if tuple(out.shape) != (B // group, Q, H * D):
            raise EvaluationError(f"out must have shape {(B // group, Q, H * D)}")
        desc.reduce_out = out.data_ptr()
        result = out
    _check_tensor(ctx, "per-entry output", torch.float32, value.device)
    if tuple(ctx.shape) != per_entry:
        raise EvaluationError(f"the per-entry buffer must have shape {per_entry}")
    table = native.int32_table(v for pair in shapes for v in pair)
    keep.append(table)
    q0, q1 = (0, Q) if q_range is None else (int(q_range[0]), int(q_range[1]))
    desc.value, desc.value_dtype = value.data_ptr(), native.GACB_F32 if value.dtype == torch.float32 else native.GACB_BF16
    desc.locations, desc.attention, desc.out = locations.data_ptr(), attention.data_ptr(), ctx.data_ptr()
    desc.spatial_hw = table
    desc.L, desc.B, desc.S, desc.Q, desc.H, desc.D, desc.P = L, B, S, Q, H, D, P
    desc.attention_is_logits = 1 if softmax else 0
    desc.group, desc.reduce_mode = group, REDUCE_MODES[reduce]
    desc.q_begin, desc.q_end = q0, q1
    if compact is not None:
        _check_tensor(compact, "compact", torch.int32, value.device)
        desc.compact_scratch, desc.compact_scratch_bytes = compact.data_ptr(), compact.numel() * 4
    with torch.cuda.device(value.device):
        rc = lib.gacb_msda_run(ctypes.byref(desc), _stream_ptr(stream))
    native.check(rc, "gacb_msda_run")
    return result


def _reuse_bits(reuse_weights: bool, reuse_input: bool, workspace, input_at_end: bool = False) -> int:
    if (reuse_weights or reuse_input or input_at_end) and workspace is None:
        raise EvaluationError("reuse_weights/reuse_input/input_at_end need the caller's workspace")
    return ((native.DCN_REUSE_WEIGHTS if reuse_weights else 0) | (native.DCN_REUSE_INPUT if reuse_input else 0)
            | (native.DCN_INPUT_AT_END if input_at_end else 0))


def workspace_parts(n, Cin, H, W, Cout, Kh, Kw, stride, pads, dilation, groups, deform_groups, math, plain=False):
    """(bytes of the channel-last input copy, bytes of the packed weights) of a DCNv2 (``plain=False``, two pads)
    or Conv2D (``plain=True``, four pads) call on ``n`` images; both 0 when the shape runs on the CUDA-core kernel."""
    pads = tuple(pads) if len(pads) == 4 else (pads[0], pads[1], pads[0], pads[1])
    copy_bytes, weight_bytes = ctypes.c_size_t(0), ctypes.c_size_t(0)
    rc = native.load().gacb_dcnv2_workspace_parts(n, Cin, H, W, Cout, Kh, Kw, stride[0], stride[1], *pads, dilation[0],
                                                  dilation[1], groups, deform_groups, native.DCN_MATH_MODES[math],
                                                  1 if plain else 0, ctypes.byref(copy_bytes), ctypes.byref(weight_bytes))
    native.check(rc, "gacb_dcnv2_workspace_parts")
    return int(copy_bytes.value), int(weight_bytes.value)


def shared_input_workspaces(x, conv_cout, dcn_cout, kernel, stride, padding, dilation, groups=1, deform_groups=1,
                            math="f32x3"):
    """One device buffer for the ``conv_offset`` -> DCNv2 pair of an R101-DCN bottleneck (both read the same ``x``):
    returns ``(buffer, conv_workspace, dcn_workspace)``, two views that end at the same address.  Call
    ``conv2d_forward(..., workspace=conv_workspace, input_at_end=True)`` first (it makes the channel-last copy of
    ``x``), then ``dcnv2_forward(..., workspace=dcn_workspace, input_at_end=True, reuse_input=True)``; add
    ``reuse_weights=True`` to both once each has packed its weights.  The block then pays for one copy, and in the
    steady state for no packing.  Returns ``(None, None, None)`` when the shapes run on the CUDA-core kernels."""
    torch = _torch()
    n, cin, h, w = x.shape
    kh, kw = kernel
    copy_c, weights_c = workspace_parts(n, cin, h, w, conv_cout, kh, kw, stride, (padding[0], padding[1]) * 2, dilation, 1,
                                        1, math, plain=True)
    copy_d, weights_d = workspace_parts(n, cin, h, w, dcn_cout, kh, kw, stride, padding, dilation, groups, deform_groups,
                                        math)
    if not copy_c or not copy_d:
        return None, None, None
    assert copy_c == copy_d, "both layers copy the same images in the same element type"
    first = -(-weights_c // 256) * 256
    total = first + -(-weights_d // 256) * 256 + copy_d
    buf = torch.empty(total, dtype=torch.uint8, device=x.device)
    return buf, buf, buf[first:]


def dcn_output_hw(H, W, Kh, Kw, stride, padding, dilation):
    Ho = (H + 2 * padding[0] - dilation[0] * (Kh - 1) - 1) // stride[0] + 1
    Wo = (W + 2 * padding[1] - dilation[1] * (Kw - 1) - 1) // stride[1] + 1
    return Ho, Wo


def dcnv2_workspace_bytes(n, Cin, H, W, Cout, Kh, Kw, stride, padding, dilation, groups, deform_groups, math):
    lib = native.load()
    return int(lib.gacb_dcnv2_workspace_bytes(n, Cin, H, W, Cout, Kh, Kw, stride[0], stride[1], padding[0],
                                              padding[1], dilation[0], dilation[1], groups, deform_groups,
                                              native.DCN_MATH_MODES[math]))


def dcnv2_forward(x, offset, mask, weight, bias=None, *, stride=(1, 1), padding=(0, 0), dilation=(1, 1),
                  groups=1, deform_groups=1, math="f32x3", out=None, n_range=None, workspace=None,
                  status_word=None, stream=None, mask_is_logits=False, batch_norm=None, relu=False, row_range=None,
                  pixel_range=None, reuse_weights=False, reuse_input=False, input_at_end=False, test_flags=0):
    """DCNv2 on device tensors (all float32, NCHW / OIHW).  ``math`` selects the
    tensor-core product: "f32x3" (fp32-faithful), "tf32" or "bf16".

    Optional neighbours folded into the kernel: ``mask_is_logits`` (the sigmoid
    that produces the mask), ``batch_norm=(scale, bias, mean, variance, epsilon)``
    (inference BatchNorm over output channels) and ``relu``.

    ``n_range=(n0, n1)`` limits the call to those images and ``row_range=(r0, r1)``
    to those output rows of each of them; ``pixel_range=(p0, p1)`` instead limits
    it to a run of the flattened (image, row, column) output pixels (one launch per
    GPU in the balanced multi-GPU split).  The rest of ``out`` is left untouched.

    ``reuse_weights`` / ``reuse_input`` promise that ``workspace`` still holds the
    packed weights / the channel-last copy of ``x`` from an earlier call (same
    tensors' contents, shapes and ``math``); the call then skips that step.
    ``test_flags`` is OR-ed into the library's ``math_mode`` argument; the only bit defined,
    ``native.DCN_TEST_DROP_WEIGHT_COPIES``, is understood by the fault-injection build alone (the normal
    library refuses it) and makes a bounded wait of the kernel run out."""
    torch = _torch()
    lib = native.load()
    if math not in native.DCN_MATH_MODES:
        raise EvaluationError(f"math must be one of {sorted(native.DCN_MATH_MODES)}")
    for t, name in ((x, "X"), (offset, "offset"), (mask, "mask"), (weight, "W")):
        _check_tensor(t, name, torch.float32, x.device if isinstance(x, torch.Tensor) else None)
        if t.dim() != 4:
            raise EvaluationError("DeformConv2D expects X/offset/mask NCHW and W OIHW rank-four tensors")
    if bias is not None:
        _check_tensor(bias, "bias", torch.float32, x.device)
    N, Cin, H, W = x.shape
    Cout, Cin_g, Kh, Kw = weight.shape
    stride, padding, dilation = tuple(stride), tuple(padding), tuple(dilation)
    if groups <= 0 or deform_groups <= 0 or Cin % groups or Cin % deform_groups or Cout % groups or Cin_g * groups != Cin:
        raise EvaluationError("DeformConv2D channels must be positive and divisible by their groups")
    if H + 2 * padding[0] < dilation[0] * (Kh - 1) + 1 or W + 2 * padding[1] < dilation[1] * (Kw - 1) + 1:
        raise EvaluationError("DeformConv2D kernel exceeds padded input")
    Ho, Wo = dcn_output_hw(H, W, Kh, Kw, stride, padding, dilation)
    K = Kh * Kw
    if tuple(offset.shape) != (N, 2 * deform_groups * K, Ho, Wo) or tuple(mask.shape) != (N, deform_groups * K, Ho, Wo):
        raise EvaluationError("DeformConv2D offset/mask shapes disagree with the output extent")
    if bias is not None and tuple(bias.shape) != (Cout,):
        raise EvaluationError("DeformConv2D bias must be [output_channels]")
    if out is None:
        out = torch.empty((N, Cout, Ho, Wo), dtype=torch.float32, device=x.device)
    n0, n1 = (0, N) if n_range is None else (int(n_range[0]), int(n_range[1]))
    if pixel_range is not None:
        if n_range is not None or row_range is not None:
            raise EvaluationError("pixel_range excludes n_range and row_range")
        p0, p1 = int(pixel_range[0]), int(pixel_range[1])
        if not 0 <= p0 <= p1 <= N * Ho * Wo:
            raise EvaluationError(f"pixel_range {pixel_range} is outside [0, {N * Ho * Wo}]")
        n0, n1 = p0 // (Ho * Wo), (p0 // (Ho * Wo) if p1 == p0 else -(-p1 // (Ho * Wo)))
    need = dcnv2_workspace_bytes(n1 - n0, Cin, H, W, Cout, Kh, Kw, stride, padding, dilation, groups,
                                 deform_groups, math)
    reuse = _reuse_bits(reuse_weights, reuse_input, workspace, input_at_end)
    if workspace is None and need:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    ws_ptr = workspace.data_ptr() if workspace is not None else None
    ws_len = workspace.numel() * workspace.element_size() if workspace is not None else 0
    dims = (N, Cin, H, W, Cout, Kh, Kw, stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1],
            groups, deform_groups, n0, n1, native.DCN_MATH_MODES[math] | reuse | int(test_flags), ws_ptr, ws_len,
            status_word.data_ptr() if status_word is not None else None, _stream_ptr(stream))
    bias_ptr = bias.data_ptr() if bias is not None else None
    if (row_range is not None or pixel_range is not None) and (mask_is_logits or batch_norm is not None or relu):
        raise EvaluationError("row_range/pixel_range cannot be combined with the folded sigmoid/BatchNorm/ReLU")
    with torch.cuda.device(x.device):
        if pixel_range is not None:
            rc = lib.gacb_dcnv2_pixels_forward(x.data_ptr(), offset.data_ptr(), mask.data_ptr(), weight.data_ptr(),
                                               bias_ptr, out.data_ptr(), *dims[:15], p0, p1, *dims[17:])
            native.check(rc, "gacb_dcnv2_pixels_forward")
        elif row_range is not None:
            r0, r1 = int(row_range[0]), int(row_range[1])
            if not 0 <= r0 <= r1 <= Ho:
                raise EvaluationError(f"row_range {row_range} is outside [0, {Ho}]")
            rc = lib.gacb_dcnv2_rows_forward(x.data_ptr(), offset.data_ptr(), mask.data_ptr(), weight.data_ptr(),
                                             bias_ptr, out.data_ptr(), *dims[:17], r0, r1, *dims[17:])
            native.check(rc, "gacb_dcnv2_rows_forward")
        elif mask_is_logits or batch_norm is not None or relu:
            bn = [None] * 4
            eps = 1e-5
            if batch_norm is not None:
                if len(batch_norm) != 5:
                    raise EvaluationError("batch_norm must be (scale, bias, mean, variance, epsilon)")
                for t, name in zip(batch_norm[:4], ("bn scale", "bn bias", "bn mean", "bn variance")):
                    _check_tensor(t, name, torch.float32, x.device)
                    if tuple(t.shape) != (Cout,):
                        raise EvaluationError("BatchNorm parameters must have shape [C]")
                bn = [t.data_ptr() for t in batch_norm[:4]]
                eps = float(batch_norm[4])
            rc = lib.gacb_dcnv2_fused_forward(x.data_ptr(), offset.data_ptr(), mask.data_ptr(),
                                              1 if mask_is_logits else 0, weight.data_ptr(), bias_ptr, *bn, eps,
                                              1 if relu else 0, out.data_ptr(), *dims)
            native.check(rc, "gacb_dcnv2_fused_forward")
        else:
            rc = lib.gacb_dcnv2_forward(x.data_ptr(), offset.data_ptr(), mask.data_ptr(), weight.data_ptr(), bias_ptr,
                                        out.data_ptr(), *dims)
            native.check(rc, "gacb_dcnv2_forward")
    return out


def conv2d_workspace_bytes(n_images, Cin, H, W, Cout, Kh, Kw, strides, pads, dilations, groups, math) -> int:
    """Scratch bytes ``conv2d_forward`` needs for ``n_images`` images (0: the CUDA-core kernel runs, no scratch)."""
    lib = native.load()
    return int(lib.gacb_conv2d_workspace_bytes(n_images, Cin, H, W, Cout, Kh, Kw, strides[0], strides[1], pads[0],
                                               pads[1], pads[2], pads[3], dilations[0], dilations[1], groups,
                                               native.DCN_MATH_MODES[math]))


def conv2d_forward(x, weight, bias=None, *, strides=(1, 1), pads=(0, 0, 0, 0), dilations=(1, 1), groups=1,
                   math="f32x3", relu=False, split_at=None, out=None, n_range=None, workspace=None,
                   status_word=None, stream=None, reuse_weights=False, reuse_input=False, input_at_end=False,
                   test_flags=0):
    """Plain convolution on device tensors (float32, NCHW / OIHW) through the DCNv2 kernels with integer taps.

    ``split_at=c`` returns two tensors, channels ``[0, c)`` and ``[c, Cout)`` -- for BEVFormer's ``conv_offset``
    (``c = 2 * deform_groups * Kh * Kw``) these are DCNv2's ``offset`` and pre-sigmoid ``mask`` operands.
    ``out`` is then a pair of tensors.  ``test_flags`` is as in ``dcnv2_forward``."""
    torch = _torch()
    lib = native.load()
    if math not in native.DCN_MATH_MODES:
        raise EvaluationError(f"math must be one of {sorted(native.DCN_MATH_MODES)}")
    for t, name in ((x, "X"), (weight, "W")):
        _check_tensor(t, name, torch.float32, x.device if isinstance(x, torch.Tensor) else None)
        if t.dim() != 4:
            raise EvaluationError("Conv2D expects NCHW input and OIHW weight")
    if bias is not None:
        _check_tensor(bias, "bias", torch.float32, x.device)
    N, Cin, H, W = x.shape
    Cout, Cin_g, Kh, Kw = weight.shape
    strides, pads, dilations = tuple(int(v) for v in strides), tuple(int(v) for v in pads), tuple(int(v) for v in dilations)
    if len(strides) != 2 or len(pads) != 4 or len(dilations) != 2 or min(strides) < 1 or min(dilations) < 1 or min(pads) < 0:
        raise EvaluationError("Conv2D needs strides/dilations pairs >= 1 and four nonnegative pads")
    if groups <= 0 or Cin % groups or Cout % groups or Cin_g * groups != Cin:
        raise EvaluationError("Conv2D channels must be divisible by groups and agree with the weights")
    if bias is not None and tuple(bias.shape) != (Cout,):
        raise EvaluationError("Conv2D bias must have shape [out_channels]")
    Ho, Wo = conv_output_hw(H, W, Kh, Kw, strides, pads, dilations)
    if Ho <= 0 or Wo <= 0:
        raise EvaluationError("convolution or pooling produces a non-positive dimension")
    if split_at is None:
        if out is None:
            out = torch.empty((N, Cout, Ho, Wo), dtype=torch.float32, device=x.device)
        y0, y1, cut = out, None, 0
    else:
        cut = int(split_at)
        if not 0 < cut < Cout:
            raise EvaluationError(f"split_at must lie inside (0, {Cout})")
        if out is None:
            out = (torch.empty((N, cut, Ho, Wo), dtype=torch.float32, device=x.device),
                   torch.empty((N, Cout - cut, Ho, Wo), dtype=torch.float32, device=x.device))
        y0, y1 = out
    for t, shape in ((y0, (N, cut or Cout, Ho, Wo)), (y1, (N, Cout - cut, Ho, Wo))):
        if t is not None:
            _check_tensor(t, "output", torch.float32, x.device)
            if tuple(t.shape) != shape:
                raise EvaluationError(f"Conv2D output must have shape {shape}")
    n0, n1 = (0, N) if n_range is None else (int(n_range[0]), int(n_range[1]))
    need = conv2d_workspace_bytes(n1 - n0, Cin, H, W, Cout, Kh, Kw, strides, pads, dilations, groups, math)
    reuse = _reuse_bits(reuse_weights, reuse_input, workspace, input_at_end)
    if workspace is None and need:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    ws_ptr = workspace.data_ptr() if workspace is not None else None
    ws_len = workspace.numel() * workspace.element_size() if workspace is not None else 0
    with torch.cuda.device(x.device):
        rc = lib.gacb_conv2d_forward(x.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None,
                                     1 if relu else 0, y0.data_ptr(), y1.data_ptr() if y1 is not None else None, cut,
                                     N, Cin, H, W, Cout, Kh, Kw, strides[0], strides[1], pads[0], pads[1], pads[2],
                                     pads[3], dilations[0], dilations[1], groups, n0, n1,
                                     native.DCN_MATH_MODES[math] | reuse | int(test_flags), ws_ptr, ws_len,
                                     status_word.data_ptr() if status_word is not None else None, _stream_ptr(stream))
        native.check(rc, "gacb_conv2d_forward")
    return out


def cast_to_bf16(t, *, stream=None):
    """float32 device tensor -> bfloat16 (round to nearest even) with the library's own kernel."""
    torch = _torch()
    lib = native.load()
    _check_tensor(t, "tensor", torch.float32)
    out = torch.empty(t.shape, dtype=torch.bfloat16, device=t.device)
    with torch.cuda.device(t.device):
        rc = lib.gacb_cast_f32_to_bf16(t.data_ptr(), out.data_ptr(), t.numel(), _stream_ptr(stream))
    native.check(rc, "gacb_cast_f32_to_bf16")
    return out


# --------------------------------------------------------------------------- #
# evaluate_op: host arrays in, host arrays out, computed on the device
# --------------------------------------------------------------------------- #

def _to_device(a, device, what: str):
    torch = _torch()
    arr = np.asarray(a)
    if not np.issubdtype(arr.dtype, np.floating):
        raise EvaluationError(f"{what} inputs must be floating point")
    if arr.dtype != np.float32:
        raise BackendError(f"{what}: this backend computes float32 tensors only, got {arr.dtype}")
    return torch.from_numpy(np.ascontiguousarray(arr)).to(device)


def evaluate_op(op: str, inputs: Sequence[np.ndarray], attrs: Mapping[str, Any] | None = None, *,
                device_id: int = 0, value_storage: str = "float32", math: str = "f32x3") -> tuple:
    """Execute one supported op on the B200; same call shape as the reference's ``evaluate_op``."""
    attrs = dict(attrs or {})
    if op not in SUPPORTED_OPS:
        raise EvaluationError(f"unsupported op {op!r}")
    device = require_device(device_id)
    torch = _torch()
    if op in ("MSDeformableAttention", "MSDeformableAttentionOffsets"):
        fused = op.endswith("Offsets")
        if len(inputs) != (5 if fused else 3):
            raise EvaluationError(f"{op} expects {'five' if fused else 'three'} inputs")
        shapes = spatial_shapes_of(attrs, EvaluationError)
        if np.asarray(inputs[0]).ndim != 4 or np.asarray(inputs[1]).ndim != 6 or np.asarray(inputs[2]).ndim != 5:
            raise EvaluationError("MSDeformableAttention expects value/location/weight ranks [4, 6, 5]")
        dev = [_to_device(a, device, op) for a in inputs]
        if value_storage == "bfloat16":
            dev[0] = cast_to_bf16(dev[0])
        elif value_storage != "float32":
            raise EvaluationError("value_storage must be 'float32' or 'bfloat16'")
        softmax = bool(attrs.get("softmax", False))
        if fused:
            out = msda_offsets_forward(dev[0], dev[1], dev[2], dev[3], dev[4], shapes,
                                       attrs.get("coordinate_shape", tuple(dev[1].shape)),
                                       bool(attrs.get("reference_first", False)), softmax=softmax)
        else:
            out = msda_forward(dev[0], dev[1], dev[2], shapes, softmax=softmax)
        torch.cuda.synchronize(device)
        return (out.cpu().numpy(),)
    if op == "Conv2D":
        if len(inputs) not in (2, 3):
            raise EvaluationError("Conv2D expects value, weight, and optional bias")
        node = Node("conv", "Conv2D", tuple(f"i{k}" for k in range(len(inputs))), ("y",), attrs)
        try:
            strides, pads, dilations, groups = conv_attrs(node)
        except ShapeInferenceError as exc:
            raise EvaluationError(str(exc)) from exc
        dev = [_to_device(a, device, op) for a in inputs]
        out = conv2d_forward(dev[0], dev[1], dev[2] if len(dev) == 3 else None, strides=strides, pads=pads,
                             dilations=dilations, groups=groups, math=math, relu=bool(attrs.get("relu", False)))
        torch.cuda.synchronize(device)
        return (out.cpu().numpy(),)
    # DeformConv2D
    if len(inputs) not in (4, 5):
        raise EvaluationError("DeformConv2D expects four or five inputs")
    node = Node("dcn", "DeformConv2D", tuple(f"i{k}" for k in range(len(inputs))), ("y",), attrs)
    try:
        stride, padding, dilation, groups, dgroups = dcn_attrs(node)
    except ShapeInferenceError as exc:
        raise EvaluationError(str(exc)) from exc
    dev = [_to_device(a, device, op) for a in inputs]
    out = dcnv2_forward(dev[0], dev[1], dev[2], dev[3], dev[4] if len(dev) == 5 else None, stride=stride,
                        padding=padding, dilation=dilation, groups=groups, deform_groups=dgroups, math=math,
                        mask_is_logits=bool(attrs.get("mask_is_logits", False)), relu=bool(attrs.get("relu", False)))
    torch.cuda.synchronize(device)
    return (out.cpu().numpy(),)
