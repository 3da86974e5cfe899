"""Graph rewriting for the deformable-sampling path.

GAC fuses a few neighbours into its sampling operators before it lowers them
(``native/lib/GraphPasses.cpp:206-271`` folds ``Div -> view -> Add -> view`` into
``gac.ms_deform_attn_offsets``; ``:338-341`` folds Conv+ReLU).  The kernels of
this library take more than that in one launch, so ``fuse_deformable_sampling``
recognises, around every ``MSDeformableAttention`` / ``DeformConv2D`` /
``Conv2D`` node, the sub-graphs BEVFormer builds there
(``src/gac/models/bevformer/spatial.py:160-188``, ``temporal.py:318-389``) and
replaces them by one node:

* ``Reshape -> Softmax(last axis) -> Reshape`` in front of the attention
  weights                                   -> attr ``softmax`` (raw scores in);
* ``Div(offsets, normalizer) -> Add(reference expanded) -> Reshape`` in front of
  the sampling locations                    -> fused coordinates;
* ``Reshape -> Mul(visibility) -> ReduceSum(axis 1) -> Div(., Clamp(ReduceSum(
  visibility), min=1))`` behind the output  -> ``reduce="masked_average"``;
* ``Reshape -> ReduceMean(axis 1)`` behind the output -> ``reduce="mean"``;
* ``Sigmoid`` in front of the DCNv2 mask, ``BatchNorm`` and ``ReLU`` behind a
  DCNv2, ``ReLU`` behind a Conv2D;
* ``Slice`` nodes along the channel axis that cut a Conv2D's output in two
  (the offsets and the mask scores that a ``conv_offset`` convolution makes
  for the DCNv2 beside it; also the three-way cut whose first two pieces are
  joined again by a ``Concat``)          -> attr ``split_at``, two outputs.

An intermediate value is only absorbed when nothing else reads it and it is not
a graph output.  What does not match is left alone; ``Reshape`` nodes that remain
are views and cost nothing at run time.
"""

from __future__ import annotations

from typing import Optional

import numpy as np

from .errors import ShapeInferenceError
from .ir import Graph, Node, TensorSpec

FUSED_MSDA = "MSDeformableAttentionFused"
ELEMENTWISE_UNARY = ("Softmax", "Sigmoid", "ReLU", "Clamp", "Identity")
ELEMENTWISE_BINARY = ("Add", "Sub", "Mul", "Div")


def _numel(shape) -> int:
    return int(np.prod(shape, dtype=np.int64)) if len(shape) else 1


def infer_neighbour_specs(graph: Graph) -> None:
    """Fill ``value_specs`` for the shape-only neighbours of the sampling operators (views, elementwise ops with
    NumPy broadcasting, reductions over listed axes); sampling operators themselves go through ``infer_node``."""
    from .ops import SUPPORTED_OPS, infer_node

    specs = graph.value_specs
    for node in graph.nodes:
        if all(o in specs for o in node.outputs):
            continue
        ins = [specs.get(n) for n in node.inputs]
        if any(s is None for s in ins):
            continue
        out: Optional[TensorSpec] = None
        if node.op in SUPPORTED_OPS or node.op == FUSED_MSDA:
            specs.update(infer_node(node, specs))
            continue
        if node.op in ("Reshape", "Expand"):
            shape = [int(d) for d in node.attrs.get("shape", ())]
            if node.op == "Reshape" and -1 in shape and ins[0].is_static:
                known = _numel([d for d in shape if d != -1])
                shape[shape.index(-1)] = ins[0].numel // max(known, 1)
            out = TensorSpec(tuple(shape), ins[0].dtype)
        elif node.op in ELEMENTWISE_UNARY or node.op == "BatchNorm":
            out = TensorSpec(ins[0].shape, ins[0].dtype)
        elif node.op == "Slice" and ins[0].is_static:
            cut = _channel_slice(node, ins[0].shape)
            if cut is not None:
                out = TensorSpec((ins[0].shape[0], cut[1] - cut[0], *ins[0].shape[2:]), ins[0].dtype)
        elif node.op == "Concat" and all(s.is_static for s in ins):
            axis = int(node.attrs.get("axis", 0)) % ins[0].rank
            shape = list(ins[0].shape)
            shape[axis] = sum(s.shape[axis] for s in ins)
            out = TensorSpec(tuple(shape), ins[0].dtype)
        elif node.op in ELEMENTWISE_BINARY and all(s.is_static for s in ins[:2]):
            out = TensorSpec(tuple(np.broadcast_shapes(ins[0].shape, ins[1].shape)), ins[0].dtype)
        elif node.op in ("ReduceSum", "ReduceMean") and ins[0].is_static:
            axes = [a % ins[0].rank for a in node.attrs.get("axes", range(ins[0].rank))]
            keep = bool(node.attrs.get("keepdims", True))
            shape = [1 if i in axes else d for i, d in enumerate(ins[0].shape) if keep or i not in axes]
            out = TensorSpec(tuple(shape), ins[0].dtype)
        elif node.op == "Transpose" and ins[0].is_static:
            perm = node.attrs.get("perm", tuple(reversed(range(ins[0].rank))))
            out = TensorSpec(tuple(ins[0].shape[p] for p in perm), ins[0].dtype)
        if out is not None:
            specs[node.outputs[0]] = out


def _channel_slice(node: Node, shape) -> Optional[tuple]:
    """``(begin, end)`` of a Slice that takes a run of whole channels (axis 1, step 1) of a rank-4 tensor and
    nothing else (the reference's attributes: starts / ends / axes / steps, src/gac/core/ops.py:262-300)."""
    starts, ends = node.attrs.get("starts"), node.attrs.get("ends")
    axes, steps = node.attrs.get("axes"), node.attrs.get("steps")
    if not isinstance(starts, (list, tuple)) or not isinstance(ends, (list, tuple)) or len(starts) != 1 or len(ends) != 1:
        return None
    axes = list(axes) if axes is not None else [0]
    steps = list(steps) if steps is not None else [1]
    if len(shape) != 4 or len(axes) != 1 or len(steps) != 1 or int(axes[0]) % 4 != 1 or int(steps[0]) != 1:
        return None
    begin, end, _ = slice(int(starts[0]), int(ends[0]), 1).indices(int(shape[1]))
    return (begin, end) if end > begin else None


class _Rewriter:
    def __init__(self, graph: Graph) -> None:
        self.g = graph
        self.producer = {o: n for n in graph.nodes for o in n.outputs}
        self.uses: dict = {}
        for n in graph.nodes:
            for i in n.inputs:
                self.uses.setdefault(i, []).append(n)
        self.dead: set = set()
        self.replaced: dict = {}
        self.details: list = []

    # ---- helpers
    def shape(self, name):
        spec = self.g.value_specs.get(name)
        return tuple(spec.shape) if spec is not None and spec.is_static else None

    def private(self, name) -> bool:
        """Read by exactly one node and not exposed by the graph."""
        return name not in self.g.outputs and len(self.uses.get(name, ())) == 1

    def made_by(self, name, op) -> Optional[Node]:
        node = self.producer.get(name)
        return node if node is not None and node.op == op and node.id not in self.dead else None

    def only_user(self, name, op) -> Optional[Node]:
        if name in self.g.outputs:
            return None
        users = self.uses.get(name, ())
        return users[0] if len(users) == 1 and users[0].op == op and users[0].id not in self.dead else None

    def through_views(self, name):
        """Walk back through private Reshape nodes; returns (root name, [view nodes])."""
        chain = []
        while True:
            node = self.made_by(name, "Reshape")
            if node is None or not self.private(name):
                return name, chain
            chain.append(node)
            name = node.inputs[0]

    def kill(self, *nodes) -> None:
        self.dead.update(n.id for n in nodes)

    # ---- MSDA
    def msda(self, node: Node) -> None:
        shapes = node.attrs.get("spatial_shapes")
        value, loc, attn = node.inputs[:3]
        loc_shape, attn_shape = self.shape(loc), self.shape(attn)
        if loc_shape is None or attn_shape is None or len(loc_shape) != 6 or len(attn_shape) != 5:
            return
        B, Q, H, L, P, _ = loc_shape
        attrs = {"spatial_shapes": shapes, "softmax": bool(node.attrs.get("softmax", False)),
                 "dims": [B, Q, H, L, P], "group": 1, "reduce": "none", "coordinates": "plain"}
        inputs = {"value": value, "locations": loc, "attention": attn}
        absorbed: list = []
        what: list = []

        # softmax over the L*P scores of a (b, q, h)
        if not attrs["softmax"] and self.private(attn):
            back = self.made_by(attn, "Reshape")
            soft = self.made_by(back.inputs[0], "Softmax") if back is not None else None
            if soft is not None and self.private(back.inputs[0]):
                s_in = self.shape(soft.inputs[0])
                axis = int(soft.attrs.get("axis", -1))
                if s_in is not None and axis % len(s_in) == len(s_in) - 1 and s_in[-1] == L * P and _numel(s_in) == B * Q * H * L * P:
                    root, views = self.through_views(soft.inputs[0])
                    inputs["attention"] = root
                    attrs["softmax"] = True
                    absorbed += [back, soft, *views]
                    what.append("softmax")

        # loc = offsets / normalizer + reference
        if self.private(loc):
            back = self.made_by(loc, "Reshape")
            add = self.made_by(back.inputs[0], "Add") if back is not None else None
            if add is not None and self.private(back.inputs[0]):
                coord = self.shape(add.outputs[0])
                for div_side in (0, 1):
                    div = self.made_by(add.inputs[div_side], "Div")
                    if div is None or not self.private(add.inputs[div_side]) or coord is None or len(coord) > 8:
                        continue
                    # the reference side: walk back through private Expand / Reshape nodes to the smallest tensor
                    # that still broadcasts against the coordinate view (the kernel does the broadcasting)
                    ref_name, ref_nodes = add.inputs[1 - div_side], []
                    cur, chain = ref_name, []
                    while True:
                        n = self.made_by(cur, "Expand") or self.made_by(cur, "Reshape")
                        if n is None or not self.private(cur):
                            break
                        chain.append(n)
                        cur = n.inputs[0]
                        if _broadcasts(self.shape(cur), coord):
                            ref_name, ref_nodes = cur, list(chain)
                    ref_shape = self.shape(ref_name)
                    if not _broadcasts(ref_shape, coord):
                        continue
                    norm_shape = self.shape(div.inputs[1])
                    merged = _merge_to_locations(norm_shape, coord, (B, Q, H, L, P, 2)) if norm_shape else None
                    if ref_shape is None or merged is None or _numel(coord) != B * Q * H * L * P * 2:
                        continue
                    off_root, off_views = self.through_views(div.inputs[0])
                    inputs.update(locations=off_root, normalizer=div.inputs[1], reference=ref_name)
                    attrs.update(coordinates="offsets", coordinate_shape=list(coord), reference_first=div_side == 1,
                                 normalizer_shape=list(merged), reference_shape=list(ref_shape))
                    absorbed += [back, add, div, *ref_nodes, *off_views]
                    what.append("coordinates")
                    break

        # what follows the output
        out_name = node.outputs[0]
        view = self.only_user(out_name, "Reshape")
        if view is not None:
            v_shape = self.shape(view.outputs[0])
            if v_shape is not None and len(v_shape) == 4 and v_shape[0] * v_shape[1] == B and v_shape[2] == Q:
                group = v_shape[1]
                mean = self.only_user(view.outputs[0], "ReduceMean")
                mul = self.only_user(view.outputs[0], "Mul")
                if mean is not None and list(mean.attrs.get("axes", ())) == [1] and not mean.attrs.get("keepdims", True):
                    attrs.update(group=group, reduce="mean")
                    absorbed += [view, mean]
                    out_name = mean.outputs[0]
                    what.append("queue mean")
                elif mul is not None:
                    vis = mul.inputs[1] if mul.inputs[0] == view.outputs[0] else mul.inputs[0]
                    total = self.only_user(mul.outputs[0], "ReduceSum")
                    div = self.only_user(total.outputs[0], "Div") if total is not None else None
                    clamp = self.made_by(div.inputs[1], "Clamp") if div is not None and div.inputs[0] == total.outputs[0] else None
                    count = self.made_by(clamp.inputs[0], "ReduceSum") if clamp is not None else None
                    vis_shape = self.shape(vis)
                    ok = (count is not None and count.inputs[0] == vis and vis_shape is not None
                          and _numel(vis_shape) == B * Q and list(total.attrs.get("axes", ())) == [1]
                          and list(count.attrs.get("axes", ())) == [1] and not total.attrs.get("keepdims", True)
                          and not count.attrs.get("keepdims", True) and float(clamp.attrs.get("min", 0)) == 1.0
                          and "max" not in clamp.attrs and self.private(clamp.outputs[0]) and self.private(count.outputs[0]))
                    if ok:
                        inputs["visibility"] = vis
                        attrs.update(group=group, reduce="masked_average")
                        absorbed += [view, mul, total, div, clamp, count]
                        out_name = div.outputs[0]
                        what.append("camera average")

        if not what:
            return
        order = ["value", "locations", "attention"] + [k for k in ("normalizer", "reference", "visibility") if k in inputs]
        attrs["operands"] = order
        fused = Node(node.id, FUSED_MSDA, tuple(inputs[k] for k in order), (out_name,), attrs,
                     tuple(dict.fromkeys(s for n in [node, *absorbed] for s in n.source_nodes)))
        self.kill(*absorbed)
        self.replaced[node.id] = fused
        self.details.append({"node": node.id, "fused": what, "removed": [n.id for n in absorbed]})

    # ---- convolutions
    def conv(self, node: Node) -> None:
        attrs = dict(node.attrs)
        inputs = list(node.inputs)
        absorbed, what = [], []
        out_name = node.outputs[0]
        if node.op == "DeformConv2D" and not attrs.get("mask_is_logits"):
            sig = self.made_by(inputs[2], "Sigmoid")
            if sig is not None and self.private(inputs[2]):
                inputs[2] = sig.inputs[0]
                attrs["mask_is_logits"] = True
                absorbed.append(sig)
                what.append("sigmoid")
        if node.op == "DeformConv2D" and not attrs.get("batch_norm") and len(inputs) == 5:
            bn = self.only_user(out_name, "BatchNorm")
            if bn is not None and bn.inputs[0] == out_name and len(bn.inputs) == 5:
                inputs += list(bn.inputs[1:])
                attrs["batch_norm"] = True
                attrs["epsilon"] = float(bn.attrs.get("epsilon", 1e-5))
                absorbed.append(bn)
                out_name = bn.outputs[0]
                what.append("batch norm")
        outputs = (out_name,)
        if node.op == "Conv2D" and attrs.get("split_at") is None:
            split = self.channel_split(out_name)
            if split is not None:
                attrs["split_at"], outputs, gone = split
                absorbed += gone
                what.append("channel split")
        if len(outputs) == 1 and not attrs.get("relu"):
            relu = self.only_user(out_name, "ReLU")
            if relu is not None:
                attrs["relu"] = True
                absorbed.append(relu)
                out_name = relu.outputs[0]
                what.append("relu")
        if not what:
            return
        if len(outputs) == 1:
            outputs = (out_name,)
        fused = Node(node.id, node.op, tuple(inputs), outputs, attrs,
                     tuple(dict.fromkeys(s for n in [node, *absorbed] for s in n.source_nodes)))
        self.kill(*absorbed)
        self.replaced[node.id] = fused
        self.details.append({"node": node.id, "fused": what, "removed": [n.id for n in absorbed]})

    def channel_split(self, name):
        """``(cut, (low output, high output), absorbed nodes)`` when the convolution output ``name`` is read only by
        Slice nodes that cut its channels into [0, cut) and [cut, C) -- two slices, or three whose first two are
        joined again, in order, by a Concat along the channels that nothing else feeds."""
        shape = self.shape(name)
        users = self.uses.get(name, ())
        if shape is None or len(shape) != 4 or name in self.g.outputs or len(users) not in (2, 3):
            return None
        cuts = []
        for user in users:
            piece = _channel_slice(user, shape) if user.op == "Slice" and user.id not in self.dead else None
            if piece is None:
                return None
            cuts.append((piece, user))
        cuts.sort(key=lambda c: c[0])
        bounds = [c[0] for c in cuts]
        if bounds[0][0] != 0 or bounds[-1][1] != shape[1] or any(a[1] != b[0] for a, b in zip(bounds, bounds[1:])):
            return None
        if len(cuts) == 2:
            return bounds[0][1], (cuts[0][1].outputs[0], cuts[1][1].outputs[0]), [cuts[0][1], cuts[1][1]]
        first, second = cuts[0][1].outputs[0], cuts[1][1].outputs[0]
        join = self.only_user(first, "Concat")
        if (join is None or self.only_user(second, "Concat") is not join or tuple(join.inputs) != (first, second)
                or int(join.attrs.get("axis", 0)) % 4 != 1):
            return None
        return bounds[1][1], (join.outputs[0], cuts[2][1].outputs[0]), [cuts[0][1], cuts[1][1], join, cuts[2][1]]


def _broadcasts(small, full) -> bool:
    if small is None or full is None or len(small) > len(full):
        return False
    padded = (1,) * (len(full) - len(small)) + tuple(small)
    return all(s == 1 or s == f for s, f in zip(padded, full))


def _merge_to_locations(norm_shape, coord, loc_shape):
    """Shape of the normaliser seen against the rank-6 location tensor, given that it broadcasts against the
    coordinate view.  The coordinate axes split into consecutive runs, one per location axis; within a run the
    normaliser must be 1 everywhere (it broadcasts over the merged axis) or full everywhere (it covers it)."""
    if not _broadcasts(norm_shape, coord):
        return None
    padded = (1,) * (len(coord) - len(norm_shape)) + tuple(norm_shape)
    merged, i = [], 0
    for want in loc_shape:
        size, ones, fulls = 1, True, True
        while size < want:
            if i >= len(coord):
                return None
            size *= coord[i]
            if coord[i] != 1:               # an axis of extent 1 says nothing either way
                ones &= padded[i] == 1
                fulls &= padded[i] == coord[i]
            i += 1
        if size != want or not (ones or fulls):
            return None
        merged.append(1 if ones else want)
    if any(d != 1 for d in coord[i:]):
        return None
    return tuple(merged)


def fuse_deformable_sampling(graph: Graph) -> tuple:
    """Returns ``(rewritten graph, report)``; the input graph is not modified."""
    g = graph.clone()
    infer_neighbour_specs(g)
    rw = _Rewriter(g)
    for node in g.nodes:
        if node.id in rw.dead:
            continue
        if node.op == "MSDeformableAttention":
            rw.msda(node)
        elif node.op in ("DeformConv2D", "Conv2D"):
            rw.conv(node)
    if not rw.replaced:
        return g, {"name": "deformable-sampling-fusion", "changed": False, "details": {"fused": []}}
    # A fused node sits where the LAST node it absorbed sat, so that every value it reads is defined before it.
    position = {n.id: k for k, n in enumerate(g.nodes)}
    last_of = {}
    for d in rw.details:
        last_of[d["node"]] = max([position[d["node"]], *[position[r] for r in d["removed"]]])
    slots: dict = {}
    for nid, fused in rw.replaced.items():
        slots[last_of[nid]] = fused
    nodes = []
    for k, node in enumerate(g.nodes):
        if k in slots:
            nodes.append(slots[k])
        elif node.id not in rw.dead and node.id not in rw.replaced:
            nodes.append(node)
    defined = {o for n in nodes for o in n.outputs} | set(g.inputs) | set(g.constants)
    specs = {k: v for k, v in g.value_specs.items() if k in defined}
    out = Graph(g.name, dict(g.inputs), g.outputs, nodes, {k: v.copy() for k, v in g.constants.items()}, specs,
                dict(g.metadata))
    try:
        out.validate()
        infer_neighbour_specs(out)
    except Exception as exc:      # a pattern that cannot be ordered: keep the original graph
        raise ShapeInferenceError(f"fusion produced an invalid graph: {exc}") from exc
    return out, {"name": "deformable-sampling-fusion", "changed": True, "details": {"fused": rw.details}}
