"""Single-device execution of a ``CudaProgram`` with host buffers at the boundary.

Same shape as the reference's ``CudaSession`` (``src/gac/execution/cuda.py``):
the constructor probes the device and allocates every device buffer once
(:140-313); ``run`` validates the host inputs, copies them to the device,
launches the planned kernels on the session's one stream, copies the outputs
back and returns a ``RunResult`` (:384-452).  A failed run invalidates the
session (:457-464) and a concurrent ``run`` raises instead of blocking
(:398-399).  There is no CPU execution path.

torch provides device memory, pinned staging buffers, the stream and events;
the kernels are reached through the C ABI (``native.py``).

Extras for measurement: ``pinned_inputs()`` exposes the session's pinned staging
arrays so a caller can fill them in place (then ``run`` copies straight from
pinned memory); ``upload`` + ``run_resident`` keep the inputs on the device
between launches.
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from threading import Lock
from typing import Any, Mapping

import numpy as np

from . import ops
from .compiler import TARGET, VIEW_OPS, CudaProgram, KernelLaunch
from .errors import BackendError, DeviceUnavailableError, ValidationError
from .ops import FUSED_MSDA, conv_attrs, dcn_attrs
from .profiler import Profiler
from .validation import all_finite, bind_inputs, checked_copy, parallel_copy


@dataclass
class RunResult:
    outputs: dict
    wall_ms: float
    gpu_stream_ms: float
    kernel_ms: float | None
    profiler: Profiler


def cuda_device_info(device_id: int = 0) -> dict[str, Any]:
    """Device facts, or ``DeviceUnavailableError``."""
    device = ops.require_device(device_id)
    import torch

    props = torch.cuda.get_device_properties(device)
    return {
        "device_id": device_id,
        "name": props.name,
        "compute_capability": [props.major, props.minor],
        "total_memory_bytes": int(props.total_memory),
        "multiprocessor_count": int(props.multi_processor_count),
        "supported_target": TARGET if props.major == 10 else None,
    }


class CudaSession:
    """Owns the device buffers and one stream; invocations are serial."""

    def __init__(self, program: CudaProgram, *, device_id: int = 0, check_finite: bool = True,
                 fresh_outputs: bool = True, overlap_batches: bool = False, cuda_graph: bool = False) -> None:
        if not isinstance(program, CudaProgram):
            raise ValidationError("CudaSession needs a CudaProgram from compile_cuda")
        self.program = program
        self.device_id = int(device_id)
        self._check_finite = bool(check_finite)
        # False: run() returns views of the pinned output buffers (valid until the next run) instead of copies
        self._fresh_outputs = bool(fresh_outputs)
        # True: a graph that is one float32 MSDeformableAttention node runs batch entry by batch entry, with the
        # host->device copy of entry b+1, the kernel of entry b and the device->host copy of entry b-1 on three
        # streams (PCIe is full duplex; the entries are independent).  Results are bit-identical to one launch.
        self._overlap_batches = bool(overlap_batches)
        # True: the launch sequence of the program (every buffer is owned by the session, so every pointer is fixed)
        # is captured into a CUDA graph on the second invocation and replayed from then on: one submission instead
        # of one Python + ctypes call per launch.  The first invocation runs eagerly; it sets the kernels' attributes
        # and packs constant weights, which the captured sequence then leaves out.  Traced / profiled invocations
        # always run launch by launch.
        self._use_graph = bool(cuda_graph)
        self._graph = None
        self._eager_runs = 0
        self._lock = Lock()
        self._closed = False
        self._failed = False
        self._device = ops.require_device(self.device_id)
        import torch

        self._torch = torch
        g = program.graph
        self._node_ops = {n.id: n for n in g.nodes}
        try:
            with torch.cuda.device(self._device):
                self._stream = torch.cuda.Stream(device=self._device)
                self._h2d_stream = torch.cuda.Stream(device=self._device)
                self._d2h_stream = torch.cuda.Stream(device=self._device)
                self._pinned = {k: torch.empty(s.shape, dtype=torch.float32).pin_memory() for k, s in g.inputs.items()}
                self._inputs = {k: torch.empty(s.shape, dtype=torch.float32, device=self._device)
                                for k, s in g.inputs.items()}
                self._constants = {k: torch.from_numpy(np.ascontiguousarray(v)).to(self._device)
                                   for k, v in g.constants.items()}
                self._values = {}
                for node in g.nodes:
                    for out in node.outputs:
                        spec = g.value_specs[out]
                        if node.op in VIEW_OPS:      # a view of its input's buffer: nothing to launch, nothing to copy
                            self._values[out] = self._lookup(node.inputs[0]).view(spec.shape)
                        else:
                            self._values[out] = torch.empty(spec.shape, dtype=torch.float32, device=self._device)
                self._scratch = {}
                self._pinned_out = {k: torch.empty(g.value_specs[k].shape, dtype=torch.float32).pin_memory()
                                    for k in g.outputs}
                self._bf16_value = {}
                self._workspaces = {}
                self._weights_packed = set()   # nodes whose constant weights are already packed in their workspace
                self._status = torch.zeros(1, dtype=torch.int32, device=self._device)
                for node in g.nodes:
                    if node.op.startswith("MSDeformableAttention") and program.options.get("value_storage") == "bfloat16":
                        spec = g.value_specs[node.inputs[0]]
                        self._bf16_value[node.id] = torch.empty(spec.shape, dtype=torch.bfloat16, device=self._device)
                    if node.op == FUSED_MSDA:
                        b, q, h, _, _ = node.attrs["dims"]
                        d = g.value_specs[node.inputs[0]].shape[3]
                        entry = {}
                        if node.attrs.get("reduce", "none") != "none":
                            entry["context"] = torch.empty((b, q, h * d), dtype=torch.float32, device=self._device)
                        if "visibility" in node.attrs["operands"]:
                            entry["compact"] = torch.empty(b * q + 4, dtype=torch.int32, device=self._device)
                        self._scratch[node.id] = entry
                        if program.options.get("value_storage") == "bfloat16":
                            spec = g.value_specs[node.inputs[0]]
                            self._bf16_value[node.id] = torch.empty(spec.shape, dtype=torch.bfloat16, device=self._device)
                    if node.op == "Conv2D":
                        x = g.value_specs[node.inputs[0]]
                        w = g.value_specs[node.inputs[1]]
                        strides, pads, dilations, groups = conv_attrs(node)
                        need = ops.conv2d_workspace_bytes(x.shape[0], x.shape[1], x.shape[2], x.shape[3], w.shape[0],
                                                          w.shape[2], w.shape[3], strides, pads, dilations, groups,
                                                          program.options.get("dcn_math", "f32x3"))
                        self._workspaces[node.id] = (torch.empty(max(need, 16), dtype=torch.uint8, device=self._device)
                                                     if need else None)
                    if node.op == "DeformConv2D":
                        x = g.value_specs[node.inputs[0]]
                        w = g.value_specs[node.inputs[3]]
                        stride, padding, dilation, groups, dgroups = dcn_attrs(node)
                        need = ops.dcnv2_workspace_bytes(x.shape[0], x.shape[1], x.shape[2], x.shape[3], w.shape[0],
                                                         w.shape[2], w.shape[3], stride, padding, dilation, groups,
                                                         dgroups, program.options.get("dcn_math", "f32x3"))
                        self._workspaces[node.id] = (torch.empty(max(need, 16), dtype=torch.uint8, device=self._device)
                                                     if need else None)
            self._share_input_copies(g, program.options.get("dcn_math", "f32x3"))
            self._pinned_np = {k: t.numpy() for k, t in self._pinned.items()}
        except DeviceUnavailableError:
            raise
        except Exception as exc:  # allocation failure, driver trouble
            raise BackendError(f"cannot open a CUDA session on device {device_id}: {exc}") from exc

    # ------------------------------------------------------------------ helpers
    def pinned_inputs(self) -> dict:
        """NumPy views of the pinned staging buffers (fill in place, then pass them to ``run``)."""
        return dict(self._pinned_np)

    @staticmethod
    def _fresh_copy(staged: np.ndarray) -> np.ndarray:
        out = np.empty_like(staged)
        parallel_copy(out, staged)
        return out

    def _lookup(self, name: str):
        if name in self._inputs:
            return self._inputs[name]
        if name in self._constants:
            return self._constants[name]
        return self._values[name]

    def _reuse_weights(self, node, weight_name: str) -> bool:
        """Weights that are graph constants never change between runs: pack them on the first launch only."""
        return (weight_name in self._constants and node.id in self._weights_packed
                and self._workspaces.get(node.id) is not None)

    def _stage_and_upload(self, name: str, arr: np.ndarray) -> None:
        """Host array -> pinned staging buffer (checked for non-finite values on the way when the session checks: one
        pass over the input instead of a check and a copy) -> device; the host->device copy of one input runs while
        the next one is staged.  (Staging and uploading slab by slab along the first axis was measured slower:
        41 ms against 24 ms per run of the base spatial workload.)"""
        staged = self._pinned_np[name]
        if arr.ctypes.data == staged.ctypes.data:                   # the caller filled the pinned view itself
            if self._check_finite and not all_finite(arr):
                raise ValidationError(f"input {name!r} must contain finite values")
        elif self._check_finite:
            checked_copy(staged, arr, name)
        else:
            parallel_copy(staged, arr)
        self._inputs[name].copy_(self._pinned[name], non_blocking=True)

    def _share_input_copies(self, g, math: str) -> None:
        """Convolutions of the graph that read the same input tensor (the ``conv_offset`` convolution and the DCNv2 it
        feeds, in every R101-DCN bottleneck) share one channel-last copy of it: their workspaces become views of one
        buffer that end at the same address, the first of them in graph order makes the copy and the others are told
        that it is there (``GACB_DCN_INPUT_AT_END`` / ``GACB_DCN_REUSE_INPUT`` of the C ABI)."""
        torch = self._torch
        self._input_copy = {}          # node id -> "make" | "reuse"
        by_input: dict = {}
        for node in g.nodes:
            if node.op not in ("Conv2D", "DeformConv2D") or self._workspaces.get(node.id) is None:
                continue
            x = g.value_specs[node.inputs[0]]
            if node.op == "Conv2D":
                w = g.value_specs[node.inputs[1]]
                strides, pads, dilations, groups = conv_attrs(node)
                parts = ops.workspace_parts(*x.shape, w.shape[0], w.shape[2], w.shape[3], strides, pads, dilations, groups, 1,
                                            math, plain=True)
            else:
                w = g.value_specs[node.inputs[3]]
                stride, padding, dilation, groups, dgroups = dcn_attrs(node)
                parts = ops.workspace_parts(*x.shape, w.shape[0], w.shape[2], w.shape[3], stride, padding, dilation, groups,
                                            dgroups, math)
            if parts[0]:
                by_input.setdefault((node.inputs[0], parts[0]), []).append((node.id, parts[1]))
        for (_, copy_bytes), members in by_input.items():
            if len(members) < 2:
                continue
            starts, at = [], 0
            for _, weight_bytes in members:
                starts.append(at)
                at += -(-weight_bytes // 256) * 256
            buffer = torch.empty(at + copy_bytes, dtype=torch.uint8, device=self._device)
            for i, ((node_id, _), start) in enumerate(zip(members, starts)):
                self._workspaces[node_id] = buffer[start:]
                self._input_copy[node_id] = "make" if i == 0 else "reuse"

    def _input_copy_flags(self, node) -> dict:
        role = self._input_copy.get(node.id)
        return {} if role is None else {"input_at_end": True, "reuse_input": role == "reuse"}

    def _implementation_for(self, launch: KernelLaunch) -> str:
        return launch.implementation_candidates[0] if launch.implementation_candidates else "unknown"

    def _execute_launch(self, launch: KernelLaunch) -> None:
        node = self._node_ops[launch.node_id]
        args = [self._lookup(n) for n in node.inputs]
        out = self._values[launch.output]
        opts = self.program.options
        if node.op == "Conv2D":
            strides, pads, dilations, groups = conv_attrs(node)
            split = node.attrs.get("split_at")
            if split is not None:
                out = (out, self._values[launch.extra_outputs[0]])
            ops.conv2d_forward(args[0], args[1], args[2] if len(args) == 3 else None, strides=strides, pads=pads,
                               dilations=dilations, groups=groups, math=opts.get("dcn_math", "f32x3"), out=out,
                               split_at=split,
                               relu=bool(node.attrs.get("relu", False)), workspace=self._workspaces.get(node.id),
                               status_word=self._status, stream=self._stream,
                               reuse_weights=self._reuse_weights(node, node.inputs[1]), **self._input_copy_flags(node))
            self._weights_packed.add(node.id)
            return
        if node.op == FUSED_MSDA:
            a = node.attrs
            b, q, h, l, p = a["dims"]
            by = dict(zip(a["operands"], args))
            value = by["value"]
            if node.id in self._bf16_value:
                lib = ops.native.load()
                rc = lib.gacb_cast_f32_to_bf16(value.data_ptr(), self._bf16_value[node.id].data_ptr(), value.numel(),
                                               int(self._stream.cuda_stream))
                ops.native.check(rc, "gacb_cast_f32_to_bf16")
                value = self._bf16_value[node.id]
            fused_coords = a.get("coordinates") == "offsets"
            scratch = self._scratch.get(node.id, {})
            ops.msda_group_forward(
                value, by["locations"].view(b, q, h, l, p, 2), by["attention"].view(b, q, h, l, p), a["spatial_shapes"],
                group=int(a.get("group", 1)), reduce=a.get("reduce", "none"),
                visibility=by["visibility"].view(b, q) if "visibility" in by else None, softmax=bool(a.get("softmax", False)),
                normalizer=by["normalizer"].view(a["normalizer_shape"]) if fused_coords else None,
                reference=by["reference"].view(a["reference_shape"]) if fused_coords else None,
                coordinate_shape=a.get("coordinate_shape") if fused_coords else None,
                reference_first=bool(a.get("reference_first", False)), scratch=scratch.get("context"), out=out,
                stream=self._stream, compact=scratch.get("compact"))
            return
        if node.op == "DeformConv2D":
            stride, padding, dilation, groups, dgroups = dcn_attrs(node)
            batch_norm = (*args[5:9], float(node.attrs.get("epsilon", 1e-5))) if node.attrs.get("batch_norm") else None
            ops.dcnv2_forward(args[0], args[1], args[2], args[3], args[4] if len(args) >= 5 else None,
                              stride=stride, padding=padding, dilation=dilation, groups=groups,
                              deform_groups=dgroups, math=opts.get("dcn_math", "f32x3"), out=out,
                              workspace=self._workspaces.get(node.id), status_word=self._status,
                              stream=self._stream, mask_is_logits=bool(node.attrs.get("mask_is_logits", False)),
                              relu=bool(node.attrs.get("relu", False)), batch_norm=batch_norm,
                              reuse_weights=self._reuse_weights(node, node.inputs[3]),
                              test_flags=int(opts.get("dcn_test_flags", 0)), **self._input_copy_flags(node))
            self._weights_packed.add(node.id)
            return
        value = args[0]
        if node.id in self._bf16_value:
            lib = ops.native.load()
            rc = lib.gacb_cast_f32_to_bf16(value.data_ptr(), self._bf16_value[node.id].data_ptr(), value.numel(),
                                           int(self._stream.cuda_stream))
            ops.native.check(rc, "gacb_cast_f32_to_bf16")
            value = self._bf16_value[node.id]
        if node.op == "MSDeformableAttention":
            ops.msda_forward(value, args[1], args[2], node.attrs["spatial_shapes"], out=out, stream=self._stream,
                             softmax=bool(node.attrs.get("softmax", False)))
        else:
            ops.msda_offsets_forward(value, args[1], args[2], args[3], args[4], node.attrs["spatial_shapes"],
                                     node.attrs.get("coordinate_shape", tuple(args[1].shape)),
                                     bool(node.attrs.get("reference_first", False)), out=out, stream=self._stream,
                                     softmax=bool(node.attrs.get("softmax", False)))

    def _launch_all(self, profiler: Profiler, instrument: bool, event_pairs: list) -> None:
        torch = self._torch
        if self._use_graph and not instrument:
            if self._graph is None and self._eager_runs >= 1:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=self._stream, capture_error_mode="thread_local"):
                    for launch in self.program.launches:
                        self._execute_launch(launch)
                self._graph = graph
            if self._graph is not None:
                self._graph.replay()
                return
            self._eager_runs += 1
        for launch in self.program.launches:
            spec = self.program.graph.value_specs[launch.output]
            meta = {"node_id": launch.node_id, "entry_point": launch.entry_point,
                    "op": self._node_ops[launch.node_id].op, "implementation": self._implementation_for(launch),
                    "grid": launch.grid, "block": launch.block, "clock": "host submission",
                    "output_bytes": spec.nbytes}
            pair = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) if instrument else None
            if pair:
                pair[0].record(self._stream)
            with profiler.record("dispatch", launch.entry_point, TARGET, source_nodes=launch.source_nodes,
                                 metadata=meta) as ev:
                self._execute_launch(launch)
            if pair:
                pair[1].record(self._stream)
                event_pairs.append((pair, ev.metadata))

    def _check_device_status(self, word: int | None = None) -> None:
        """Map the device status word to the reference's failure contract: a kernel that gave up a bounded wait
        left incomplete outputs, so the invocation raises ``BackendError`` and the session is invalid from then on
        (``src/gac/execution/cuda.py:457-464``).  ``word`` overrides the device read (host-side tests)."""
        if word is None:
            word = int(self._status.item())
        rc = ops.native.load().gacb_status_from_word(int(word))
        if rc != ops.native.GACB_OK:
            self._failed = True
            ops.native.check(rc, "device status word")

    def _can_overlap(self) -> bool:
        g = self.program.graph
        if not self._overlap_batches or len(g.nodes) != 1 or self.program.options.get("value_storage") != "float32":
            return False
        node = g.nodes[0]
        return (node.op == "MSDeformableAttention" and set(node.inputs) == set(g.inputs)
                and g.outputs == node.outputs and g.inputs[node.inputs[0]].shape[0] > 1)

    def _run_overlapped(self, bound) -> float:
        """Batch-entry pipeline over three streams; returns the device milliseconds from first copy to last."""
        torch = self._torch
        node = self.program.graph.nodes[0]
        value, loc, attn = (self._inputs[n] for n in node.inputs)
        pv, pl, pa = (self._pinned[n] for n in node.inputs)
        out = self._values[node.outputs[0]]
        pout = self._pinned_out[node.outputs[0]]
        for name, arr in bound.items():
            staged = self._pinned_np[name]
            if arr.ctypes.data != staged.ctypes.data:
                parallel_copy(staged, arr)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # everything queued earlier on the compute stream (a previous run reading these buffers) comes first
        self._h2d_stream.wait_stream(self._stream)
        self._d2h_stream.wait_stream(self._stream)
        start.record(self._h2d_stream)
        batch = value.shape[0]
        for b in range(batch):
            with torch.cuda.stream(self._h2d_stream):
                value[b].copy_(pv[b], non_blocking=True)
                loc[b].copy_(pl[b], non_blocking=True)
                attn[b].copy_(pa[b], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(self._h2d_stream)
            self._stream.wait_event(arrived)
            ops.msda_forward(value[b:b + 1], loc[b:b + 1], attn[b:b + 1], node.attrs["spatial_shapes"],
                             out=out[b:b + 1], stream=self._stream, softmax=bool(node.attrs.get("softmax", False)))
            done = torch.cuda.Event()
            done.record(self._stream)
            with torch.cuda.stream(self._d2h_stream):
                self._d2h_stream.wait_event(done)
                pout[b].copy_(out[b], non_blocking=True)
        end.record(self._d2h_stream)
        self._d2h_stream.synchronize()
        self._stream.synchronize()
        return float(start.elapsed_time(end))

    # ------------------------------------------------------------------ public API
    def run(self, inputs: Mapping[str, np.ndarray], *, trace: bool = False, profile: bool = False) -> RunResult:
        """One invocation: validate, host->device, launches, device->host (fresh host arrays)."""
        if not self._lock.acquire(blocking=False):
            raise BackendError("concurrent calls on a single CUDA Session are not supported")
        try:
            if self._closed or self._failed:
                raise BackendError("CUDA Session is closed or failed; create a new Session")
            started = time.perf_counter()
            torch = self._torch
            instrument = trace or profile
            overlapped = not instrument and self._can_overlap()
            # Names, shapes, dtypes and contiguity first.  The finite check of the general path rides on the staging
            # copy below (one pass over the inputs instead of two); no kernel is launched before every input passed.
            bound = bind_inputs(self.program.graph, inputs, check_finite=self._check_finite and overlapped)
            profiler = Profiler(enabled=instrument)
            event_pairs: list = []
            if overlapped:
                with torch.cuda.device(self._device):
                    gpu_ms = self._run_overlapped(bound)
                    outputs = {name: (self._fresh_copy(self._pinned_out[name].numpy()) if self._fresh_outputs
                                      else self._pinned_out[name].numpy())
                               for name in self.program.graph.outputs}
                return RunResult(outputs, (time.perf_counter() - started) * 1000.0, gpu_ms, None, profiler)
            with torch.cuda.device(self._device), torch.cuda.stream(self._stream):
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record(self._stream)
                nbytes = sum(v.nbytes for v in bound.values())
                with profiler.record("copy_h2d", "inputs", TARGET, metadata={"bytes": nbytes, "clock": "host submission"}):
                    for name, arr in bound.items():
                        self._stage_and_upload(name, arr)
                self._launch_all(profiler, instrument, event_pairs)
                end.record(self._stream)
                with profiler.record("copy_d2h", "outputs", TARGET, metadata={"clock": "host including completion wait"}):
                    for name in self.program.graph.outputs:
                        self._pinned_out[name].copy_(self._lookup(name), non_blocking=True)
                    self._stream.synchronize()
                    outputs = {name: (self._fresh_copy(self._pinned_out[name].numpy()) if self._fresh_outputs
                                      else self._pinned_out[name].numpy())
                               for name in self.program.graph.outputs}
                self._check_device_status()
                gpu_ms = float(start.elapsed_time(end))
                kernel_ms = None
                if instrument:
                    kernel_ms = 0.0
                    for pair, meta in event_pairs:
                        meta["gpu_elapsed_ms"] = float(pair[0].elapsed_time(pair[1]))
                        kernel_ms += meta["gpu_elapsed_ms"]
            return RunResult(outputs, (time.perf_counter() - started) * 1000.0, gpu_ms, kernel_ms, profiler)
        except (ValidationError, BackendError):
            raise
        except Exception as exc:
            self._failed = True
            raise BackendError(f"CUDA invocation failed; Session is invalidated: {exc}") from exc
        finally:
            self._lock.release()

    def upload(self, inputs: Mapping[str, np.ndarray]) -> None:
        """Validate and copy the inputs to the device once (for ``run_resident``)."""
        bound = bind_inputs(self.program.graph, inputs, check_finite=self._check_finite)
        torch = self._torch
        with self._lock, torch.cuda.device(self._device), torch.cuda.stream(self._stream):
            for name, arr in bound.items():
                parallel_copy(self._pinned_np[name], arr)
                self._inputs[name].copy_(self._pinned[name], non_blocking=True)
            self._stream.synchronize()

    def run_resident(self, repeats: int = 1) -> list:
        """Launch the program ``repeats`` times on device-resident inputs; per-repeat device ms (CUDA events)."""
        if self._closed or self._failed:
            raise BackendError("CUDA Session is closed or failed; create a new Session")
        torch = self._torch
        times = []
        with self._lock, torch.cuda.device(self._device), torch.cuda.stream(self._stream):
            profiler = Profiler(False)
            pairs = []
            for _ in range(int(repeats)):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(self._stream)
                self._launch_all(profiler, False, [])
                b.record(self._stream)
                pairs.append((a, b))
            self._stream.synchronize()
            self._check_device_status()
            times = [float(a.elapsed_time(b)) for a, b in pairs]
        return times

    def device_output(self, name: str):
        """The device tensor holding a graph output (valid until the next run)."""
        return self._lookup(name)

    def close(self) -> None:
        with self._lock:
            if self._closed:
                return
            try:
                self._stream.synchronize()
            finally:
                self._graph = None
                for store in (self._pinned, self._inputs, self._constants, self._values, self._pinned_out,
                              self._bf16_value, self._workspaces, self._pinned_np):
                    store.clear()
                self._closed = True

    def __enter__(self) -> "CudaSession":
        return self

    def __exit__(self, *_: Any) -> None:
        self.close()
