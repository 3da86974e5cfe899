#!/usr/bin/env python3
"""Benchmark of the deformable-sampling hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload base_sca]

One *step* is one pass of multi-scale deformable attention over one batch of
synthetic BEVFormer-base spatial-cross-attention input (6 cameras, 4 levels,
S=30825, H=8, D=32, L=4, P=8, Q=10000 queries per camera = 15.36 M bilinear
samples).  The metric is G bilinear samples/s (one sample = one (b,q,h,l,p)
tuple: 4 taps x D channels).

``value``     device-resident inputs, CUDA events around the K launches.
``e2e``       the same metric through ``CudaSession.run`` with pinned HOST
              buffers: host->device copies of value/locations/weights and the
              device->host copy of the output are inside the timed region.
``roofline``  algorithmic bytes per launch / average launch time against the
              measured HBM copy bandwidth; beside it the tap bytes the kernel
              gathers per second against the random-line gather rate that the
              library's probe kernel measures in the same run.
``dcnv2``     the DCNv2 stage shapes c4 / c5 in the three math modes (TFLOP/s
              against the measured bf16 tensor peak), the conv_offset
              convolution, the chain conv_offset -> DCNv2 + sigmoid +
              BatchNorm + ReLU, and the same with weights packed beforehand.
``other_msda``  the remaining MSDA configurations, CUDA-graph timed.
``cpu_baseline``  the NumPy restatement of the reference evaluator, timed on
              this host on a bounded sample of the same workload.

Multi-GPU (torchrun, one rank per GPU): "strong" scaling of the same step.  The
10000 queries per camera are cut into N blocks, rank r owns block r of every
camera; ``value`` is the whole job's samples over the slowest rank's time with
the value tensor already replicated in each GPU's own memory (one NCCL
broadcast, timed apart as ``value_broadcast_ms``).  ``with_value_replication``
times the step with the replication inside it, pipelined per camera on a
communication stream: broadcast from rank 0, and all-gather of a value that
starts out S-sharded, in float32 and bfloat16.  ``e2e`` at N > 1 is
``distributed.ShardedMsda.step``: a rank uploads 1/N of value and its own
query block from pinned host memory, the ranks all-gather value over NVLink.

``--impl reference`` times the reference's CPU implementation of the same path
(its own NumPy evaluator from the git-ignored oracle/_ref when present, else its
restatement under oracle/) with every host thread, and the reference CLI's
single-thread loop beside it.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "BEVFormer-base SCA MSDA Gsamples/s"
UNIT = "Gsamples/s"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of msda_rows_kernel on the base_sca workload: constants
# taken from one ncu capture of a full-size launch, not measured by this run (ncu cannot run inside a timed bench).
NCU_TRAFFIC_BYTES = {"float32": 467_982_336, "bfloat16": 350_548_736}
NCU_TRAFFIC_SOURCE = "constant from an ncu capture (one full-size launch, 2026-11-25), not measured in this run"


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Polls SM clock and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, device_index: int) -> None:
        self.samples: list[tuple[int, int]] = []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._handle = None
        try:
            import pynvml
            import torch

            pynvml.nvmlInit()
            self._nv = pynvml
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self._handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self._handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._handle = None

    def _loop(self) -> None:
        nv = self._nv
        while not self._stop.is_set():
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                self.samples.append((mhz, reasons))
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self._handle is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *_):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        seen = 0
        for _, r in self.samples:
            seen |= r
        reasons = [k for k, bit in names.items() if seen & bit]
        mhz = sorted(m for m, _ in self.samples)
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(mhz)}


def measured_tensor_peak() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["bf16_tflops"]), "measured bf16 burst"
    except Exception:
        return 1590.0, "fallback bf16 burst"


def measure_tf32_peak(device, n: int = 8192, reps: int = 10) -> float:
    """TFLOP/s of the library's TF32 GEMM (torch.matmul on float32 operands with TF32 products allowed), n^3,
    best of `reps` single launches timed with CUDA events: the denominator for the TF32 mode of DCNv2, measured the
    way the bf16 figure in MEASURED_PEAKS.json was (burst)."""
    import torch

    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn((n, n), device=device)
        b = torch.randn((n, n), device=device)
        c = torch.empty((n, n), device=device)
        for _ in range(3):
            torch.matmul(a, b, out=c)
        best = float("inf")
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b, out=c)
            e1.record()
            torch.cuda.synchronize(device)
            best = min(best, e0.elapsed_time(e1))
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def measure_gather_rate(device, buffer_mb: float, launches: int = 10, lane_bytes: int = 16) -> float:
    """GB/s at which all SMs gather random 128-byte lines from a buffer of `buffer_mb` MB (the library's probe
    kernel: 16-byte loads, eight lanes per line, sixteen in flight -- the MSDA tap-gather access shape alone)."""
    import ctypes

    import torch

    from general_ai_compiler_b200 import native

    lib = native.load()
    buf = torch.empty(int(buffer_mb * (1 << 20)), dtype=torch.uint8, device=device).random_(0, 255)
    sink = torch.zeros(1, dtype=torch.int32, device=device)
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    gathered = ctypes.c_size_t(0)
    stream = torch.cuda.current_stream(device)

    def launch():
        rc = lib.gacb_gather_probe(buf.data_ptr(), buf.numel(), sms * 8, 256, lane_bytes, 12345, sink.data_ptr(),
                                   ctypes.byref(gathered), ctypes.c_void_p(stream.cuda_stream))
        if rc != 0:
            raise RuntimeError(native.last_error())

    for _ in range(3):
        launch()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    a.record(stream)
    for _ in range(launches):
        launch()
    b.record(stream)
    torch.cuda.synchronize(device)
    return gathered.value * launches / (a.elapsed_time(b) * 1e-3) / 1e9


def dcn_cpu_baseline(wl) -> dict:
    """The C restatement of GAC's DCNv2 lowering on this host, one camera of the workload: one thread and every
    core (OpenMP), plus torchvision's CPU operator (the reference's own golden source) when it is importable."""
    from general_ai_compiler_b200.bevformer import make_workload_inputs
    from oracle import dcnv2_c

    x = {k: v[:1] if k in ("X", "offset", "mask") else v for k, v in make_workload_inputs(wl).items()}
    flops = wl.flops / wl.batch
    kw = dict(stride=wl.stride, padding=wl.padding, dilation=wl.dilation, groups=wl.groups, deform_groups=wl.deform_groups)
    res = {"kind": "port", "unit": "TFLOP/s", "sample": f"1 of {wl.batch} cameras of {wl.name}, C restatement of the lowering"}
    for label, threads in (("all_cores", host_threads()), ("one_core", 1)):
        if threads > 1:
            dcnv2_c(x["X"], x["offset"], x["mask"], x["W"], x["bias"], threads=threads, **kw)   # warm-up
        t0 = time.perf_counter()
        dcnv2_c(x["X"], x["offset"], x["mask"], x["W"], x["bias"], threads=threads, **kw)
        res[label] = {"cores": threads, "tflops": flops / (time.perf_counter() - t0) / 1e12}
    try:
        import torch
        import torchvision

        t = {k: torch.from_numpy(v) for k, v in x.items()}
        with torch.inference_mode():
            fn = lambda: torchvision.ops.deform_conv2d(t["X"], t["offset"], t["W"], t["bias"], stride=wl.stride,
                                                       padding=wl.padding, dilation=wl.dilation, mask=t["mask"])
            fn()
            t0 = time.perf_counter()
            fn()
        res["torchvision_cpu"] = {"cores": torch.get_num_threads(), "tflops": flops / (time.perf_counter() - t0) / 1e12,
                                  "version": torchvision.__version__}
    except Exception as exc:      # a courtesy number: its absence is not an error
        res["torchvision_cpu"] = {"unavailable": type(exc).__name__}
    return res


def bench_dcn(device, keys=("dcn_c4", "dcn_c5"), modes=("f32x3", "tf32", "bf16"), steps: int = 20, warmup: int = 3,
              world: int = 1, rank: int = 0, reduce_max=None, barrier=None, cpu_baseline: bool = False) -> dict:
    """DCNv2 (R101-DCN stage shapes, 6 cameras): device-resident launches (NHWC copy + weight packing + implicit
    GEMM per call), CUDA events on the launching stream; TFLOP/s and fraction of the bf16 tensor peak.

    With ``world > 1`` the six cameras are split two ways, every rank holding X/W in its own memory, the time the
    max over ranks and the TFLOP/s the whole job's ("strong" scaling: six cameras in total):
    the balanced split into equal runs of output pixels, one launch per rank (the main figure), the same balance
    as (camera, output-row block) pieces (``row_block_split``, up to three launches per rank), and the literal split
    into contiguous camera blocks (``camera_split``; ranks beyond the sixth idle)."""
    import torch

    from general_ai_compiler_b200 import ops
    from general_ai_compiler_b200.bevformer import WORKLOADS, make_workload_inputs

    from general_ai_compiler_b200.distributed import dcn_pixel_block, dcn_rank_pieces, unit_block

    peak, peak_kind = measured_tensor_peak()
    tf32_peak = measure_tf32_peak(device)
    out = {"unit": "TFLOP/s", "peak": peak, "peak_source": peak_kind, "tf32_peak": tf32_peak,
           "tf32_peak_source": "torch.matmul fp32 8192^3 with TF32 products, best of 10, measured in this run"}
    if world > 1:
        out["sharding"] = (f"equal runs of output pixels over {world} ranks, one launch per rank; row_block_split = "
                           "(camera, output-row block) pieces; camera_split = contiguous camera blocks; time = max over ranks")
    stream = torch.cuda.current_stream()
    for key in keys:
        wl = WORKLOADS[key]
        t = {k: torch.from_numpy(v).to(device) for k, v in make_workload_inputs(wl).items()}
        ho, wo = wl.out_hw
        y = torch.empty((wl.batch, wl.cout, ho, wo), dtype=torch.float32, device=device)
        n0, n1 = unit_block(wl.batch, world, rank)
        splits = {"": [(n0, n1, None)]}
        if world > 1:
            splits = {"": [("pixels", dcn_pixel_block(wl.batch, ho * wo, world, rank), None)],
                      "/row_block_split": [(p0, p1, (r0, r1)) for p0, p1, r0, r1 in dcn_rank_pieces(wl.batch, ho, world, rank)],
                      "/camera_split": [(n0, n1, None)]}
        if world == 1 and cpu_baseline:
            out[f"{key}/cpu_baseline"] = dcn_cpu_baseline(wl)
        for math in modes:
            # a rank's share touches at most ceil(cameras / world) + 1 images (a pixel run may straddle cameras)
            need = ops.dcnv2_workspace_bytes(min(wl.batch, -(-wl.batch // world) + 1), wl.cin, wl.height, wl.width, wl.cout, wl.kernel[0], wl.kernel[1],
                                             wl.stride, wl.padding, wl.dilation, wl.groups, wl.deform_groups, math)
            ws = torch.empty(max(need, 16), dtype=torch.uint8, device=device)
            status = torch.zeros(1, dtype=torch.int32, device=device)
            for suffix, pieces in splits.items():

                def launch():
                    for p0, p1, rows in pieces:
                        if p0 == "pixels":
                            if p1[1] > p1[0]:
                                ops.dcnv2_forward(t["X"], t["offset"], t["mask"], t["W"], t["bias"], stride=wl.stride,
                                                  padding=wl.padding, dilation=wl.dilation, math=math, out=y, workspace=ws,
                                                  status_word=status, stream=stream, pixel_range=p1)
                        elif p1 > p0:
                            ops.dcnv2_forward(t["X"], t["offset"], t["mask"], t["W"], t["bias"], stride=wl.stride,
                                              padding=wl.padding, dilation=wl.dilation, math=math, out=y, workspace=ws,
                                              status_word=status, stream=stream, n_range=(p0, p1), row_range=rows)

                for _ in range(warmup):
                    launch()
                torch.cuda.synchronize()
                if barrier is not None:
                    barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                for _ in range(steps):
                    launch()
                b.record(stream)
                torch.cuda.synchronize()
                if int(status.item()) != 0:
                    raise SystemExit("DCNv2 kernel reported an expired wait")
                ms = a.elapsed_time(b) / steps
                if reduce_max is not None:
                    ms = reduce_max(ms)
                tf = wl.flops / (ms * 1e-3) / 1e12
                out[f"{key}/{math}{suffix}"] = {"ms": ms, "tflops": tf, "frac_of_bf16_peak": tf / peak}
                if math == "tf32":
                    out[f"{key}/{math}{suffix}"]["frac_of_tf32_peak"] = tf / tf32_peak
            if world == 1:
                # the convolution that produces the offsets and mask scores (27 channels, split into the two DCNv2
                # operands), and the bottleneck chain conv_offset -> DCNv2 with sigmoid, BatchNorm and ReLU folded in
                k2 = wl.kernel[0] * wl.kernel[1]
                w_off = (torch.randn((3 * k2, wl.cin, *wl.kernel), device=device) * (2.0 / (k2 * wl.cin)) ** 0.5).contiguous()
                b_off = torch.zeros(3 * k2, device=device)
                pads = (wl.padding[0], wl.padding[1], wl.padding[0], wl.padding[1])
                off_out = (torch.empty_like(t["offset"]), torch.empty_like(t["mask"]))
                need_c = ops.conv2d_workspace_bytes(wl.batch, wl.cin, wl.height, wl.width, 3 * k2, wl.kernel[0], wl.kernel[1],
                                                    wl.stride, pads, wl.dilation, 1, math)
                ws_c = torch.empty(max(need_c, 16), dtype=torch.uint8, device=device)
                bn = tuple(torch.rand(wl.cout, device=device) + 0.5 for _ in range(4)) + (1e-5,)

                def conv_offset(workspace=ws_c, **reuse):
                    ops.conv2d_forward(t["X"], w_off, b_off, strides=wl.stride, pads=pads, dilations=wl.dilation, math=math,
                                       split_at=2 * k2, out=off_out, workspace=workspace, status_word=status, stream=stream,
                                       **reuse)

                def dcn_fused(**reuse):
                    ops.dcnv2_forward(t["X"], off_out[0], off_out[1], t["W"], t["bias"], stride=wl.stride, padding=wl.padding,
                                      dilation=wl.dilation, math=math, out=y, workspace=ws, status_word=status, stream=stream,
                                      mask_is_logits=True, batch_norm=bn, relu=True, **reuse)

                def chain():
                    conv_offset()
                    dcn_fused()

                def chain_steady():
                    # inference steady state: both sets of weights were packed by an earlier step and stay in their
                    # own workspaces; each call still copies X channel-last into its workspace
                    conv_offset(reuse_weights=True)
                    dcn_fused(reuse_weights=True)

                # one buffer for the pair: the channel-last copy of X at its end, shared; each layer's weights in front
                _, ws_conv_shared, ws_dcn_shared = ops.shared_input_workspaces(t["X"], 3 * k2, wl.cout, wl.kernel, wl.stride,
                                                                               wl.padding, wl.dilation, wl.groups,
                                                                               wl.deform_groups, math)

                def chain_shared(**reuse):
                    ops.conv2d_forward(t["X"], w_off, b_off, strides=wl.stride, pads=pads, dilations=wl.dilation, math=math,
                                       split_at=2 * k2, out=off_out, workspace=ws_conv_shared, status_word=status,
                                       stream=stream, input_at_end=True, **reuse)
                    ops.dcnv2_forward(t["X"], off_out[0], off_out[1], t["W"], t["bias"], stride=wl.stride, padding=wl.padding,
                                      dilation=wl.dilation, math=math, out=y, workspace=ws_dcn_shared, status_word=status,
                                      stream=stream, mask_is_logits=True, batch_norm=bn, relu=True, input_at_end=True,
                                      reuse_input=True, **reuse)

                def chain_shared_steady():
                    chain_shared(reuse_weights=True)

                def dcn_prepacked():
                    ops.dcnv2_forward(t["X"], t["offset"], t["mask"], t["W"], t["bias"], stride=wl.stride, padding=wl.padding,
                                      dilation=wl.dilation, math=math, out=y, workspace=ws, status_word=status, stream=stream,
                                      reuse_weights=True)

                def dcn_kernel_alone():
                    # the tensor-core kernel by itself: weights packed and the channel-last copy already in the
                    # workspace (as for the second call of the chain, which shares conv_offset's copy)
                    ops.dcnv2_forward(t["X"], t["offset"], t["mask"], t["W"], t["bias"], stride=wl.stride, padding=wl.padding,
                                      dilation=wl.dilation, math=math, out=y, workspace=ws, status_word=status, stream=stream,
                                      reuse_weights=True, reuse_input=True)

                def conv_offset_gather_kernel():
                    # the same call with the window kernel switched off: the gather kernel on integer taps
                    before = ops.native.load().gacb_conv_window_path(0)
                    try:
                        conv_offset()
                    finally:
                        ops.native.load().gacb_conv_window_path(before)

                for name, fn, flops in (("conv_offset", conv_offset, 2.0 * wl.batch * 3 * k2 * wl.cin * k2 * ho * wo),
                                        ("conv_offset/gather_kernel", conv_offset_gather_kernel,
                                         2.0 * wl.batch * 3 * k2 * wl.cin * k2 * ho * wo),
                                        ("conv_offset+dcn+bn+relu", chain, None),
                                        ("conv_offset+dcn+bn+relu/weights_prepacked", chain_steady, None),
                                        ("conv_offset+dcn+bn+relu/shared_input_copy", chain_shared, None),
                                        ("conv_offset+dcn+bn+relu/shared_input_copy+weights_prepacked", chain_shared_steady, None),
                                        ("weights_prepacked", dcn_prepacked, float(wl.flops)),
                                        ("kernel_alone", dcn_kernel_alone, float(wl.flops))):
                    for _ in range(warmup):
                        fn()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize()
                    a.record(stream)
                    for _ in range(steps):
                        fn()
                    b.record(stream)
                    torch.cuda.synchronize()
                    if int(status.item()) != 0:
                        raise SystemExit("convolution kernel reported an expired wait")
                    ms = a.elapsed_time(b) / steps
                    entry = {"ms": ms}
                    if flops:
                        entry["tflops"] = flops / (ms * 1e-3) / 1e12
                    if name == "kernel_alone":
                        entry["frac_of_bf16_peak"] = entry["tflops"] / peak
                        if math == "tf32":
                            entry["frac_of_tf32_peak"] = entry["tflops"] / tf32_peak
                    out[f"{key}/{math}/{name}"] = entry
    return out


def bench_other_msda(device, steps: int = 30, warmup: int = 5) -> dict:
    """The other MSDA configurations (device-resident, CUDA events): temporal self-attention, the tiny profiles, the
    decoder's 900-query cross-attention, and the all-query spatial cross-attention block with sparse visibility."""
    import torch

    from general_ai_compiler_b200 import ops
    from general_ai_compiler_b200.bevformer import WORKLOADS, MsdaWorkload, make_workload_inputs

    peak, _ = measured_peaks()
    stream = None      # the library call picks up torch's current stream (the capturing one inside a graph)
    out = {"timing": "CUDA graph of %d calls, replayed once, CUDA events around the replay" % steps}

    def timed(fn):
        """Average device time of one call.  The calls are captured into one CUDA graph and replayed, so that a
        kernel of a few microseconds is not timed at the pace of the host's launch path."""
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for _ in range(steps):
                    fn()
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    cases = {k: WORKLOADS[k] for k in ("base_tsa", "tiny_sca", "tiny_tsa")}
    cases["decoder_cross_attention"] = MsdaWorkload("decoder", 1, 900, 8, 32, 4, ((50, 50),), "uniform", 0.0, 20261131)
    for key, w in cases.items():
        t = {k: torch.from_numpy(v).to(device) for k, v in make_workload_inputs(w).items()}
        y = torch.empty((w.batch, w.queries, w.heads * w.head_dim), dtype=torch.float32, device=device)
        vb = ops.cast_to_bf16(t["value"])
        for label, v, item in (("f32", t["value"], 4), ("bf16_value", vb, 2)):
            ms = timed(lambda: ops.msda_forward(v, t["sampling_locations"], t["attention_weights"], w.spatial_shapes,
                                                out=y, stream=stream))
            out[f"{key}/{label}"] = {"us": ms * 1e3, "gsamples_per_s": w.samples / (ms * 1e-3) / 1e9,
                                     "hbm_frac": w.algorithmic_bytes(item) / (ms * 1e-3) / 1e9 / peak}
    # spatial cross-attention with every BEV query kept per camera (Q=40000) and ~25 % of (camera, query) pairs
    # visible: dense MSDA + masking afterwards (what the reference's graph does) against row-skip + camera average.
    w = WORKLOADS["base_sca"].with_queries(40000)
    t = {k: torch.from_numpy(v).to(device) for k, v in make_workload_inputs(w).items()}
    vis = (torch.rand((1, w.batch, w.queries, 1), device=device, generator=torch.Generator(device).manual_seed(3))
           < 0.25).float().contiguous()
    ctx = torch.empty((w.batch, w.queries, 256), dtype=torch.float32, device=device)
    red = torch.empty((1, w.queries, 256), dtype=torch.float32, device=device)
    dense_ms = timed(lambda: ops.msda_forward(t["value"], t["sampling_locations"], t["attention_weights"],
                                              w.spatial_shapes, out=ctx, stream=stream))
    skip_ms = timed(lambda: ops.msda_group_forward(t["value"], t["sampling_locations"], t["attention_weights"],
                                                   w.spatial_shapes, group=w.batch, reduce="masked_average",
                                                   visibility=vis, scratch=ctx, out=red, stream=stream))
    compact = torch.empty(w.batch * w.queries + 4, dtype=torch.int32, device=device)
    compact_ms = timed(lambda: ops.msda_group_forward(t["value"], t["sampling_locations"], t["attention_weights"],
                                                      w.spatial_shapes, group=w.batch, reduce="masked_average",
                                                      visibility=vis, scratch=ctx, out=red, stream=stream,
                                                      compact=compact))
    out["sca_all_queries_q40000_visible25pct"] = {
        "dense_msda_only_us": dense_ms * 1e3, "row_skip_plus_camera_average_us": skip_ms * 1e3,
        "compacted_rows_plus_camera_average_us": compact_ms * 1e3,
        "visible_fraction": float(vis.mean().item()), "samples_dense": w.samples}
    # base spatial cross-attention through the fused entry points: raw scores and raw offsets in, softmax and
    # coordinate arithmetic in the kernel (the same sampling positions and weights as the headline launch), and the
    # whole block with visibility (all visible) and the camera average behind it
    w = WORKLOADS["base_sca"]
    x = make_workload_inputs(w)
    loc = x["sampling_locations"]                                                        # [B,Q,H,L,P,2]
    norm = np.asarray([[ww, hh] for hh, ww in w.spatial_shapes], np.float32).reshape(1, 1, 1, w.levels, 1, 2)
    ref = loc.mean(axis=(2, 3, 4), keepdims=True).astype(np.float32)                     # [B,Q,1,1,1,2]
    offs = ((loc - ref) * norm).astype(np.float32)
    logits = np.log(np.maximum(x["attention_weights"], 1e-30)).astype(np.float32)
    t = {k: torch.from_numpy(np.ascontiguousarray(v)).to(device) for k, v in
         (("value", x["value"]), ("loc", loc), ("attn", x["attention_weights"]), ("offs", offs), ("logits", logits),
          ("norm", norm), ("ref", ref))}
    y = torch.empty((w.batch, w.queries, w.heads * w.head_dim), dtype=torch.float32, device=device)
    red = torch.empty((1, w.queries, w.heads * w.head_dim), dtype=torch.float32, device=device)
    vis = torch.ones((1, w.batch, w.queries, 1), dtype=torch.float32, device=device)
    coord = (w.batch, w.queries, w.heads, w.levels, w.points, 2)
    plain_ms = timed(lambda: ops.msda_forward(t["value"], t["loc"], t["attn"], w.spatial_shapes, out=y, stream=stream))
    fused_ms = timed(lambda: ops.msda_offsets_forward(t["value"], t["offs"], t["logits"], t["norm"], t["ref"],
                                                      w.spatial_shapes, coord, out=y, stream=stream, softmax=True))
    block_ms = timed(lambda: ops.msda_group_forward(t["value"], t["offs"], t["logits"], w.spatial_shapes, group=w.batch,
                                                    reduce="masked_average", visibility=vis, softmax=True,
                                                    normalizer=t["norm"], reference=t["ref"], coordinate_shape=coord,
                                                    scratch=y, out=red, stream=stream))
    sparse = (torch.rand((1, w.batch, w.queries, 1), device=device, generator=torch.Generator(device).manual_seed(5))
              < 0.25).float().contiguous()
    sparse_list = torch.empty(w.batch * w.queries + 4, dtype=torch.int32, device=device)
    block_kw = dict(group=w.batch, reduce="masked_average", softmax=True, normalizer=t["norm"], reference=t["ref"],
                    coordinate_shape=coord, scratch=y, out=red, stream=stream)
    skip25_ms = timed(lambda: ops.msda_group_forward(t["value"], t["offs"], t["logits"], w.spatial_shapes,
                                                     visibility=sparse, **block_kw))
    compact25_ms = timed(lambda: ops.msda_group_forward(t["value"], t["offs"], t["logits"], w.spatial_shapes,
                                                        visibility=sparse, compact=sparse_list, **block_kw))
    out["base_sca_fused_forms"] = {
        "block_25pct_visible_row_skip_us": skip25_ms * 1e3, "block_25pct_visible_compacted_us": compact25_ms * 1e3,
        "locations_and_weights_us": plain_ms * 1e3, "offsets_and_scores_in_kernel_us": fused_ms * 1e3,
        "block_with_visibility_and_camera_average_us": block_ms * 1e3,
        "note": "same sampling positions and weights in all three; the reference runs Softmax, Div, Add, Mul, "
                "ReduceSum, Clamp and Div as separate operators around the first"}
    # the public session API on device-resident inputs: launch by launch against CUDA-graph replay (wall time per
    # invocation of the program's launch sequence; the decoder program is one 8-us kernel, the DCN block three)
    from general_ai_compiler_b200.bevformer import build_dcn_block_graph, build_dcn_bottleneck_graph, build_msda_graph_for
    from general_ai_compiler_b200.compiler import compile_cuda
    from general_ai_compiler_b200.session import CudaSession

    def block_inputs(wl):
        x = make_workload_inputs(wl)
        rng = np.random.default_rng(7)
        bn = {f"bn_{p}": rng.uniform(0.5, 1.5, wl.cout).astype(np.float32) for p in ("scale", "bias", "mean", "variance")}
        return {"X": x["X"], "offset": x["offset"], "mask_scores": x["mask"], "W": x["W"], "bias": x["bias"], **bn}

    programs = {"decoder_cross_attention": (build_msda_graph_for(cases["decoder_cross_attention"]),
                                            make_workload_inputs(cases["decoder_cross_attention"])),
                "dcn_c4_block": (build_dcn_block_graph(WORKLOADS["dcn_c4"]), block_inputs(WORKLOADS["dcn_c4"]))}
    # the whole deformable stage of a bottleneck as an exporter writes it (conv_offset -> Slice x3 -> Concat ->
    # Sigmoid -> DeformConv2D -> BatchNorm -> ReLU, weights as graph constants): two launches and one channel-last copy
    def bottleneck(wl):
        x = block_inputs(wl)
        rng = np.random.default_rng(9)
        k3 = 3 * wl.kernel[0] * wl.kernel[1]
        constants = {"W_offset": (rng.standard_normal((k3, wl.cin, *wl.kernel)) * (2.0 / (9 * wl.cin)) ** 0.5).astype(np.float32),
                     "b_offset": np.zeros(k3, np.float32), "W": x["W"], "bias": x["bias"],
                     **{k: v for k, v in x.items() if k.startswith("bn_")}}
        return build_dcn_bottleneck_graph(wl, constants, three_way=True), {"X": x["X"]}

    math_of = {}
    for math in ("f32x3", "tf32", "bf16"):
        programs[f"dcn_c4_bottleneck/{math}"] = bottleneck(WORKLOADS["dcn_c4"])
        math_of[f"dcn_c4_bottleneck/{math}"] = math
    replay = {}
    for key, (graph, inputs) in programs.items():
        program = compile_cuda(graph, dcn_math=math_of.get(key, "f32x3"))
        row = {}
        for label, use_graph in (("launch_by_launch_us", False), ("cuda_graph_us", True)):
            with CudaSession(program, device_id=device.index or 0, check_finite=False, cuda_graph=use_graph) as session:
                session.upload(inputs)
                session.run_resident(3)
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                session.run_resident(100)
                row[label] = (time.perf_counter() - t0) / 100 * 1e6
        replay[key] = row
    out["session_run_resident"] = replay
    return out


def host_threads() -> int:
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def _reference_evaluator():
    """(callable(value, loc, attn, shapes) -> out, kind, what): the reference's own NumPy evaluator when the
    git-ignored copy under oracle/_ref exists (made by oracle/make_ref.py from a checkout), else its restatement."""
    import oracle

    if oracle.reference_available():
        ref = oracle.load_reference()

        def run(value, loc, attn, shapes):
            return ref.evaluate_op("MSDeformableAttention", [value, loc, attn], {"spatial_shapes": [list(s) for s in shapes]})[0]

        return run, "reference", "the reference's own gac.core.ops.evaluate_op"
    from oracle.msda_numpy import msda_forward

    return msda_forward, "port", "NumPy restatement of the reference evaluator (oracle/_ref absent)"


def _over_threads(fn, value, loc, attn, shapes, threads: int):
    """`fn` on (batch entry, query block) pieces spread over host threads (NumPy's gather loops drop the GIL);
    every output element is produced by the evaluator's own arithmetic, pieces never share one."""
    from concurrent.futures import ThreadPoolExecutor

    n_batch, n_query = loc.shape[0], loc.shape[1]
    per_batch = max(1, -(-threads // n_batch))
    step = max(1, -(-n_query // per_batch))
    jobs = [(b, q0, min(n_query, q0 + step)) for b in range(n_batch) for q0 in range(0, n_query, step)]
    out = np.empty((n_batch, n_query, value.shape[2] * value.shape[3]), np.float32)

    def run(job):
        b, q0, q1 = job
        out[b:b + 1, q0:q1] = fn(value[b:b + 1], np.ascontiguousarray(loc[b:b + 1, q0:q1]),
                                 np.ascontiguousarray(attn[b:b + 1, q0:q1]), shapes)

    with ThreadPoolExecutor(max_workers=max(1, threads)) as pool:
        list(pool.map(run, jobs))
    return out


def _sample_of(workload, total_queries: int):
    cams = max(1, min(workload.batch, total_queries // workload.queries))
    q_per_cam = min(workload.queries, max(1, total_queries // cams))
    return type(workload)(workload.name, cams, q_per_cam, workload.heads, workload.head_dim, workload.points,
                          workload.spatial_shapes, workload.location_model, workload.sigma, workload.seed)


def cpu_reference_throughput(workload, seconds_budget: float, steps: int, warmup: int, single_thread_seconds: float = 0.0):
    """Times the reference's CPU implementation of the path on a bounded sample of the workload.

    Main figure: the evaluator given every host thread (query blocks in parallel).  Beside it, when
    ``single_thread_seconds`` > 0, the figure of the reference's own command line -- one process, one thread,
    ``reference_run`` in a ``perf_counter`` loop (src/gac/tools/cli.py:764-771).

    Returns a dict: rate (samples/s), times_ms, sample, cores, kind, and optionally single_thread."""
    from general_ai_compiler_b200.bevformer import make_workload_inputs

    fn, kind, what = _reference_evaluator()
    threads = host_threads()
    probe = _sample_of(workload, 256)
    x = make_workload_inputs(probe)
    args = (x["value"], x["sampling_locations"], x["attention_weights"], probe.spatial_shapes)
    _over_threads(fn, *args, threads=threads)
    t0 = time.perf_counter()
    _over_threads(fn, *args, threads=threads)
    rate = probe.samples / (time.perf_counter() - t0)
    per_step = seconds_budget / max(1, steps + warmup)
    per_query = workload.heads * workload.levels * workload.points
    q = int(max(threads * 16, min(workload.queries * workload.batch, rate * per_step / per_query)))
    sample = _sample_of(workload, q)
    x = make_workload_inputs(sample)
    args = (x["value"], x["sampling_locations"], x["attention_weights"], sample.spatial_shapes)
    for _ in range(warmup):
        _over_threads(fn, *args, threads=threads)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        _over_threads(fn, *args, threads=threads)
        times.append(time.perf_counter() - t0)
    res = {"rate": sample.samples * steps / sum(times), "times_ms": [t * 1e3 for t in times], "cores": threads, "kind": kind,
           "sample": f"{sample.batch} camera(s) x {sample.queries} queries of {workload.name} per step "
                     f"({sample.samples} samples), {what}, query blocks over {threads} host threads"}
    if single_thread_seconds > 0:
        res["single_thread"] = cpu_reference_cli_loop(workload, single_thread_seconds)
    return res


def cpu_reference_cli_loop(workload, seconds_budget: float) -> dict:
    """One process, one thread: ``reference_run(graph, inputs)`` timed the way the reference's CLI times its
    ``numpy-cpu`` backend (one warm-up, then ``perf_counter`` around each call; src/gac/tools/cli.py:764-771),
    on a sample sized to the budget.  Falls back to the restated evaluator when oracle/_ref is absent."""
    import oracle
    from general_ai_compiler_b200.bevformer import make_workload_inputs

    fn, kind, what = _reference_evaluator()
    rate_guess = 0.6e6                                       # samples/s of the NumPy loop on one core, roughly
    per_query = workload.heads * workload.levels * workload.points
    sample = _sample_of(workload, int(max(64, min(workload.queries * workload.batch, rate_guess * seconds_budget / 3 / per_query))))
    x = make_workload_inputs(sample)
    if kind == "reference":
        ref = oracle.load_reference()
        graph = oracle.reference_msda_graph(ref, sample.batch, sample.spatial_size, sample.queries, sample.heads,
                                            sample.head_dim, sample.levels, sample.points, sample.spatial_shapes)
        call = lambda: ref.reference_run(graph, x)
        what = "the reference's own reference_run (input validation + evaluate_node)"
    else:
        call = lambda: fn(x["value"], x["sampling_locations"], x["attention_weights"], sample.spatial_shapes)
    call()
    times = []
    for _ in range(2):
        t0 = time.perf_counter()
        call()
        times.append(time.perf_counter() - t0)
    return {"value": sample.samples / (sum(times) / len(times)) / 1e9, "unit": UNIT, "cores": 1, "kind": kind,
            "sample": f"{sample.batch} camera(s) x {sample.queries} queries ({sample.samples} samples), {what}"}


def run_reference_arm(args, workload) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = cpu_reference_throughput(workload, args.cpu_seconds, args.steps, args.warmup, single_thread_seconds=max(0.5, min(15.0, args.cpu_seconds / 8)))
    value = r["rate"] / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.mean(r["times_ms"])),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(workload, max(1, args.gpus)) | {"note": "CPU arm: each step is a bounded sample of the workload"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": r["cores"], "kind": r["kind"], "sample": r["sample"],
                         "single_thread_cli_loop": r.get("single_thread")},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def bench_config(workload, world: int) -> dict:
    """The `config` object both arms print (same keys, so the two lines describe one configuration)."""
    return {"workload": workload.name, "cameras": workload.batch, "global_queries_per_camera": workload.queries,
            "levels": workload.levels, "points": workload.points, "heads": workload.heads, "head_dim": workload.head_dim,
            "spatial_shapes": [list(s) for s in workload.spatial_shapes], "samples_per_step": workload.samples,
            "sharding": f"{world} query block(s) of {workload.queries} queries per camera, value replicated"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--probe-only", action="store_true",
                    help="only measure the random-line gather rates (the profiling case for the probe kernel)")
    ap.add_argument("--workload", default="base_sca",
                    choices=["base_sca", "base_tsa", "tiny_sca", "tiny_tsa", "dcn_c4", "dcn_c5"])
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the host-buffer loop (0 = min(steps, 20))")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=120.0,
                    help="--impl reference: CPU time the whole run may take; each step is a sample sized to fit it")
    ap.add_argument("--msda-tile-path", action="store_true",
                    help="let one-level raster-query workloads (base_tsa, tiny_tsa) run the shared-memory tile kernel "
                         "(gacb_msda_tile_path(1)); the profiling case for msda_tile_kernel")
    ap.add_argument("--kernel-only", action="store_true",
                    help="device-resident launches only (no host-buffer loop, no CPU baseline): the profiling case")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    from general_ai_compiler_b200.bevformer import WORKLOADS, build_msda_graph_for, make_workload_inputs

    if args.probe_only:
        import torch

        from general_ai_compiler_b200 import ops

        device = ops.require_device(0)
        torch.cuda.set_device(device)
        print(json.dumps({"gather_probe_GBps": {"random_lines_64KB_l1_resident": measure_gather_rate(device, 0.0625),
                                                "random_lines_32MB_l2_resident": measure_gather_rate(device, 32),
                                                "random_lines_256MB": measure_gather_rate(device, 256)}}), flush=True)
        return
    if args.workload.startswith("dcn"):
        # secondary workload: DCNv2 launches only (also the profiling case for dcn_umma_kernel)
        import torch

        from general_ai_compiler_b200 import ops

        device = ops.require_device(int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(device)
        print(json.dumps({"workload": args.workload, "dcnv2": bench_dcn(device, (args.workload,), steps=args.steps,
                                                                       warmup=max(1, args.warmup))}), flush=True)
        return
    workload = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, workload)
        return

    import torch
    import torch.distributed as dist

    from general_ai_compiler_b200 import ops
    from general_ai_compiler_b200.compiler import compile_cuda
    from general_ai_compiler_b200.distributed import (ShardedMsda, bind_host_near_gpu, broadcast_value, head_shard,
                                                     nccl_high_priority_options, query_block)
    from general_ai_compiler_b200.session import CudaSession

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    device = ops.require_device(local_rank)
    torch.cuda.set_device(device)
    if args.msda_tile_path:
        ops.native.load().gacb_msda_tile_path(1)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device, pg_options=nccl_high_priority_options())

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- inputs: every rank draws the same seeded tensors and keeps its own query block of locations/weights;
    # the value tensor is made on rank 0 and replicated into each GPU's own memory by one NCCL broadcast
    numa_cpus = bind_host_near_gpu(local_rank) if world > 1 else None
    q0, q1 = query_block(workload.queries, world, rank)
    local = workload.with_queries(q1 - q0)
    host = make_workload_inputs(workload)
    host["sampling_locations"] = np.ascontiguousarray(host["sampling_locations"][:, q0:q1])
    host["attention_weights"] = np.ascontiguousarray(host["attention_weights"][:, q0:q1])
    value_dev = torch.from_numpy(host["value"]).to(device) if rank == 0 else torch.empty(
        host["value"].shape, dtype=torch.float32, device=device)
    bcast_ms = 0.0
    if world > 1:
        for _ in range(2):                                   # the first broadcasts set up NCCL's channels
            broadcast_value(value_dev, src=0)
        bcast_ms = reduce_max(min(broadcast_value(value_dev, src=0) for _ in range(3)))
    loc_dev = torch.from_numpy(host["sampling_locations"]).to(device)
    attn_dev = torch.from_numpy(host["attention_weights"]).to(device)
    out_dev = torch.empty((local.batch, local.queries, local.heads * local.head_dim), dtype=torch.float32, device=device)
    value_bf16 = ops.cast_to_bf16(value_dev)
    torch.cuda.synchronize()

    stream = torch.cuda.current_stream()

    def timed_launches(value_t, steps: int, warmup: int):
        for _ in range(warmup):
            ops.msda_forward(value_t, loc_dev, attn_dev, local.spatial_shapes, out=out_dev, stream=stream)
        barrier()
        events = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        events[0].record(stream)
        for k in range(steps):
            ops.msda_forward(value_t, loc_dev, attn_dev, local.spatial_shapes, out=out_dev, stream=stream)
            events[k + 1].record(stream)
        barrier()
        total_ms = events[0].elapsed_time(events[-1])
        per = [events[k].elapsed_time(events[k + 1]) for k in range(steps)]
        return total_ms, per

    with ClockSampler(local_rank) as clocks:
        total_ms, per_launch = timed_launches(value_dev, args.steps, args.warmup)
    total_ms = reduce_max(total_ms)
    clock_summary = clocks.summary()
    total_samples = workload.samples * args.steps            # the whole job: all ranks' query blocks together
    value_gs = total_samples / (total_ms * 1e-3) / 1e9
    avg_launch_ms = float(np.mean(per_launch))

    bf_total_ms, bf_per = timed_launches(value_bf16, args.steps, max(3, args.warmup // 2))
    bf_total_ms = reduce_max(bf_total_ms)

    # ---- parity spot check of what was just timed (rank 0, a slice, against the C oracle)
    parity = None
    if rank == 0:
        from oracle import msda_c

        nq = min(64, local.queries)
        want = msda_c(host["value"], host["sampling_locations"][:, :nq], host["attention_weights"][:, :nq],
                      local.spatial_shapes)
        got = out_dev[:, :nq].float().cpu().numpy()      # out_dev holds the bf16-value run: 1e-2 gate
        ops.msda_forward(value_dev, loc_dev, attn_dev, local.spatial_shapes, out=out_dev, stream=stream)
        torch.cuda.synchronize()
        got32 = out_dev[:, :nq].cpu().numpy()
        from general_ai_compiler_b200.validation import compare_tensor

        cmp32, cmp16 = compare_tensor(got32, want), compare_tensor(got, want)
        parity = {"fp32_max_abs": float(np.abs(got32 - want).max()), "bf16_value_max_abs": float(np.abs(got - want).max()),
                  "checked": f"first {nq} queries of every camera against the C oracle",
                  "fp32": {k: getattr(cmp32, k) for k in ("max_abs", "max_rel", "cosine", "close_fraction")},
                  "bf16_value": {k: getattr(cmp16, k) for k in ("max_abs", "max_rel", "cosine", "close_fraction")}}
        if parity["fp32_max_abs"] > 1e-4:
            raise SystemExit(f"parity failure in bench: {parity}")

    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"kernel_only": True, "workload": local.name, "fp32_avg_launch_ms": avg_launch_ms,
                              "bf16_value_avg_launch_ms": float(np.mean(bf_per)), "parity": parity}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- N > 1: the step with the replication of `value` inside it.  The value starts out S-sharded (each rank
    # holds 1/N of every camera's rows, as a value projection computed in parallel would leave it) or whole on rank
    # 0; per camera it is all-gathered / broadcast over NVLink into each GPU's own memory on a communication stream
    # while the kernel gathers from the previous camera's slab.
    e2e_steps = args.e2e_steps or min(args.steps, 20)
    replication = None
    sharded_e2e = None
    if world > 1:
        full_host = make_workload_inputs(workload)
        replication = {"note": "device-resident step = per-camera collective on a communication stream + MSDA kernel on the "
                               "compute stream, camera b+1 on the wire while camera b is gathered; ms = max over ranks; "
                               "step_ms = launched from Python call by call (host-paced), step_ms_cuda_graph = the whole "
                               "step captured once into a CUDA graph and replayed; collective_only_ms = the six "
                               "collectives (or peer copies) alone, call by call; peer_copy_* = the all-gather done by the "
                               "copy engines (cudaMemcpyAsync between the ranks' memories) instead of NCCL kernels",
                       "kernel_only_ms_per_step": total_ms / args.steps}
        rep_steps = max(5, min(args.steps, 50))

        def timed_resident(runner, with_kernel: bool, graph: bool = False):
            run = runner.step_resident if with_kernel else (lambda: [runner._replicate_entry(b) for b in range(runner.B)])
            if graph:
                run = runner.capture_resident()
                ok = torch.tensor([1 if run is not None else 0], device=device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)          # every rank replays, or none does
                if int(ok.item()) == 0:
                    return None
            for _ in range(3):
                run()
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            done = torch.cuda.current_stream()
            a.record(done)
            runner.s_comm.wait_event(a)
            runner.s_compute.wait_event(a)
            for _ in range(rep_steps):
                run()
            done.wait_stream(runner.s_comm)
            done.wait_stream(runner.s_compute)
            b.record(done)
            barrier()
            return reduce_max(a.elapsed_time(b) / rep_steps)

        for label, mode, storage in (("broadcast_f32", "broadcast", "float32"), ("all_gather_f32", "all_gather", "float32"),
                                     ("all_gather_bf16", "all_gather", "bfloat16"), ("peer_copy_f32", "peer_copy", "float32"),
                                     ("peer_copy_bf16", "peer_copy", "bfloat16")):
            # Setting up the peer-copy route maps every other rank's buffers (CUDA IPC); if that fails on any rank, all
            # ranks leave the route out together and the line says why, instead of losing the whole bench line.
            failure = ""
            try:
                runner = ShardedMsda(batch=workload.batch, spatial_shapes=workload.spatial_shapes, queries=workload.queries,
                                     heads=workload.heads, head_dim=workload.head_dim, points=workload.points, device=device,
                                     value_storage=storage, replicate=mode)
            except Exception as exc:  # noqa: BLE001 - reported in the line
                if mode != "peer_copy":
                    raise
                runner, failure = None, f"{type(exc).__name__}: {exc}"
            ok = torch.tensor([0 if failure else 1], device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                replication[label] = {"unavailable": failure or "setup failed on another rank"}
                continue      # what was set up is left to process exit: closing it needs every rank
            runner.load_host(full_host["value"], full_host["sampling_locations"], full_host["attention_weights"])
            runner.upload()
            if mode == "broadcast":
                runner.set_broadcast_source(full_host["value"])
            step_ms = timed_resident(runner, True)
            coll_ms = timed_resident(runner, False)
            graph_ms = timed_resident(runner, True, graph=True)
            item = 4 if storage == "float32" else 2
            slab_bytes = workload.batch * workload.spatial_size * workload.heads * workload.head_dim * item
            recv = slab_bytes * (world - 1) / world if mode != "broadcast" else slab_bytes
            kern_ms = (total_ms if storage == "float32" else bf_total_ms) / args.steps
            best_ms = min(step_ms, graph_ms) if graph_ms else step_ms
            replication[label] = {
                "step_ms": step_ms, "step_ms_cuda_graph": graph_ms, "collective_only_ms": coll_ms,
                "gsamples_per_s": workload.samples / (best_ms * 1e-3) / 1e9,
                "received_bytes_per_rank": int(recv), "received_GBps_per_rank": recv / (coll_ms * 1e-3) / 1e9,
                "frac_of_measured_peer_copy_770GBps": recv / (coll_ms * 1e-3) / 1e9 / 770.0,
                "bound_by": "collective" if coll_ms > kern_ms else "kernel"}
            if label == "all_gather_f32":
                # the end-to-end step through host buffers: a rank uploads only its 1/N of value and its own query
                # block; the ranks all-gather value over NVLink; the host moves one copy of the inputs in total
                for _ in range(3):
                    runner.step()
                barrier()
                t0 = time.perf_counter()
                for _ in range(e2e_steps):
                    e2e_out_t = runner.step()
                barrier()
                ms = reduce_max((time.perf_counter() - t0) * 1e3)
                sharded_e2e = {"ms": ms, "h2d": runner.h2d_bytes, "d2h": runner.d2h_bytes,
                               "out": e2e_out_t.numpy().copy()}
            if mode == "peer_copy":
                # the device-side barriers never gave up (on any rank), and the slabs the copy engines assembled give
                # the oracle's result
                word = torch.tensor([int(runner.peers.status.item())], device=device)
                dist.all_reduce(word, op=dist.ReduceOp.MAX)
                if int(word.item()) != 0:
                    replication[label] = {"unavailable": f"a device-side peer barrier ran out (status {int(word.item())})"}
                    runner.close()
                    continue
                got = runner.out[:, :8].cpu().numpy()
                from oracle import msda_c

                ref_value = full_host["value"] if storage == "float32" else torch.from_numpy(full_host["value"]).to(
                    torch.bfloat16).float().numpy()
                want = msda_c(ref_value, host["sampling_locations"][:, :8], host["attention_weights"][:, :8], workload.spatial_shapes)
                if float(np.abs(got - want).max()) > 1e-4:
                    raise SystemExit(f"peer-copy replication parity failure: {float(np.abs(got - want).max())}")
                replication[label]["how"] = ("copy-engine peer copies out of CUDA-IPC-mapped shard buffers, two bounded "
                                             "device-side barriers per step; no collective kernel")
            runner.close()
            del runner
        torch.cuda.synchronize()

    # ---- N > 1, the other way to cut the step: by attention heads.  A rank keeps only its heads of value,
    # locations and weights (what head-wise projections would hand it), so nothing is replicated and nothing
    # crosses NVLink; its output is a block of columns.  Reported beside the query-block figures.
    head_split = None
    if world > 1 and workload.heads % world == 0:
        full_host = make_workload_inputs(workload)
        hv, hl, ha, (h0, h1) = head_shard(full_host["value"], full_host["sampling_locations"], full_host["attention_weights"],
                                          world, rank)
        del full_host
        hw = type(workload)(workload.name, workload.batch, workload.queries, h1 - h0, workload.head_dim, workload.points,
                            workload.spatial_shapes, workload.location_model, workload.sigma, workload.seed)
        tv, tl, ta = (torch.from_numpy(t).to(device) for t in (hv, hl, ha))
        tout = torch.empty((hw.batch, hw.queries, hw.heads * hw.head_dim), dtype=torch.float32, device=device)
        for _ in range(max(3, args.warmup)):
            ops.msda_forward(tv, tl, ta, hw.spatial_shapes, out=tout, stream=stream)
        barrier()
        a_ev, b_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a_ev.record(stream)
        for _ in range(args.steps):
            ops.msda_forward(tv, tl, ta, hw.spatial_shapes, out=tout, stream=stream)
        b_ev.record(stream)
        barrier()
        hs_ms = reduce_max(a_ev.elapsed_time(b_ev) / args.steps)
        session = CudaSession(compile_cuda(build_msda_graph_for(hw)), device_id=local_rank, check_finite=False,
                              fresh_outputs=False, overlap_batches=True)
        pinned = session.pinned_inputs()
        for name, arr in (("value", hv), ("sampling_locations", hl), ("attention_weights", ha)):
            np.copyto(pinned[name], arr)
        for _ in range(3):
            session.run(pinned)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            res = session.run(pinned)
        barrier()
        hs_e2e_ms = reduce_max((time.perf_counter() - t0) * 1e3) / e2e_steps
        hs_err = None
        if rank == 0:
            from oracle import msda_c

            want = msda_c(hv, hl[:, :16], ha[:, :16], hw.spatial_shapes)
            hs_err = float(np.abs(res.outputs["output"][:, :16] - want).max())
            if hs_err > 1e-4:
                raise SystemExit(f"head-split parity failure in bench: max abs {hs_err}")
        session.close()
        head_split = {"heads_per_gpu": h1 - h0, "ms_per_step": hs_ms, "value": workload.samples / (hs_ms * 1e-3) / 1e9,
                      "unit": UNIT, "value_bytes_per_gpu": int(hv.nbytes), "collectives": "none",
                      "e2e": {"value": workload.samples / (hs_e2e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": hs_e2e_ms,
                              "h2d_bytes_per_step": int(hv.nbytes + hl.nbytes + ha.nbytes),
                              "d2h_bytes_per_step": int(tout.numel() * 4), "checked_max_abs": hs_err,
                              "path": "CudaSession.run on the rank's heads (stripped session, per-camera pipeline)"}}
        del tv, tl, ta, tout

    # ---- end to end
    if world == 1:
        # CudaSession.run with pinned host buffers, the stripped session (no finite check, outputs returned as views)
        graph = build_msda_graph_for(local)
        session = CudaSession(compile_cuda(graph), device_id=local_rank, check_finite=False, fresh_outputs=False,
                              overlap_batches=True)
        pinned = session.pinned_inputs()
        for name, arr in host.items():
            np.copyto(pinned[name], arr)
        h2d = sum(int(a.nbytes) for a in pinned.values())
        d2h = int(out_dev.numel() * 4)
        for _ in range(3):
            session.run(pinned)
        barrier()
        t0 = time.perf_counter()
        gpu_ms = 0.0
        for _ in range(e2e_steps):
            res = session.run(pinned)
            gpu_ms += res.gpu_stream_ms
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        e2e_out = res.outputs["output"]
        session.close()
        # the same through the session with the reference's defaults: finite check of every input and fresh host
        # copies of the outputs (src/gac/validation/reference.py:14-29, src/gac/execution/cuda.py:441-443)
        default_steps = max(2, min(5, e2e_steps))
        with CudaSession(compile_cuda(graph), device_id=local_rank) as session:
            session.run(host)
            t0 = time.perf_counter()
            for _ in range(default_steps):
                session.run(host)
            default_ms = (time.perf_counter() - t0) * 1e3 / default_steps
        e2e_extra = {"device_ms_per_step": gpu_ms / e2e_steps,
                     "default_session": {"ms_per_step": default_ms, "value": workload.samples / (default_ms * 1e-3) / 1e9,
                                         "unit": UNIT, "note": "check_finite=True, fresh output copies, pageable caller arrays"}}
        e2e_how = ("CudaSession.run, check_finite=False, fresh_outputs=False, overlap_batches=True (per-camera copy/compute/"
                   "copy pipeline, 6 launches per step), pinned staging filled in place")
    else:
        e2e_ms, h2d, d2h = sharded_e2e["ms"], sharded_e2e["h2d"], sharded_e2e["d2h"]
        e2e_out = sharded_e2e["out"]
        e2e_extra = {"host_bytes_per_step_all_ranks": (h2d + d2h) * world, "numa_bound_cpus": len(numa_cpus) if numa_cpus else None}
        e2e_how = ("distributed.ShardedMsda.step: per camera, each rank uploads its 1/N of the value rows and its own "
                   "query block from pinned host memory, all-gathers the slab over NVLink, runs the kernel, copies its "
                   "output block back; four streams")
    e2e_gs = workload.samples * e2e_steps / (e2e_ms * 1e-3) / 1e9
    if rank == 0:
        from oracle import msda_c

        nq = min(16, local.queries)
        want = msda_c(host["value"], host["sampling_locations"][:, :nq], host["attention_weights"][:, :nq], local.spatial_shapes)
        e2e_err = float(np.abs(np.asarray(e2e_out)[:, :nq] - want).max())
        if e2e_err > 1e-4:
            raise SystemExit(f"end-to-end parity failure in bench: max abs {e2e_err}")

    # DCNv2 (secondary workload): all ranks take part so that the max over ranks is a collective
    dcn_result = bench_dcn(device, world=world, rank=rank, cpu_baseline=world == 1,
                           reduce_max=reduce_max if world > 1 else None,
                           barrier=barrier if world > 1 else None)

    if rank == 0:
        peak, peak_kind = measured_peaks()
        alg_bytes = local.algorithmic_bytes(4)
        achieved = alg_bytes / (avg_launch_ms * 1e-3) / 1e9
        bf_avg = float(np.mean(bf_per))
        gather_bytes = local.samples * 4 * local.head_dim * 4
        # the gather roof: random-line rate from an L2-resident buffer (one camera's value is 31.6 MB) and from a
        # buffer as large as the whole value tensor (larger than L2)
        gather_peak_l2 = measure_gather_rate(device, 32)
        gather_peak_big = measure_gather_rate(device, 256)
        gather_peak_l1 = measure_gather_rate(device, 0.0625)                     # 64 KB: every line hits in L1
        config = bench_config(workload, world)
        config.update({"queries_per_camera_per_gpu": local.queries, "samples_per_step_per_gpu": local.samples,
                       "l2": "inputs (435 MB per step at one GPU; the 189 MB value alone at any N) larger than L2 "
                             "(126 MB); no flush",
                       "e2e_path": e2e_how})
        line = {
            "metric": METRIC, "value": value_gs, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config,
            "e2e": {"value": e2e_gs, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps, "checked_max_abs": e2e_err, **e2e_extra},
            "gpu_launches": args.steps,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_BYTES["float32"] if world == 1 else None,
                         "traffic_source": NCU_TRAFFIC_SOURCE if world == 1 else "not captured for a query block",
                         "peak_source": f"{peak_kind} copy bandwidth",
                         "kernel": "msda_rows_kernel<float,4,8>", "algorithmic_bytes_per_launch": alg_bytes,
                         "avg_launch_ms": avg_launch_ms, "min_launch_ms": float(np.min(per_launch)),
                         "median_launch_ms": float(np.median(per_launch)),
                         "gather_bytes_per_launch": gather_bytes,
                         "gather_achieved_GBps": gather_bytes / (avg_launch_ms * 1e-3) / 1e9,
                         "gather_peak_GBps": {"random_lines_32MB_l2_resident": gather_peak_l2,
                                              "random_lines_256MB": gather_peak_big,
                                              "random_lines_64KB_l1_resident": gather_peak_l1,
                                              "source": "gacb_gather_probe measured in this run"},
                         "gather_frac_of_l2_resident_peak": gather_bytes / (avg_launch_ms * 1e-3) / 1e9 / gather_peak_l2},
            "bf16_value": {"value": workload.samples * args.steps / (bf_total_ms * 1e-3) / 1e9, "unit": UNIT,
                           "avg_launch_ms": bf_avg,
                           "roofline_frac": local.algorithmic_bytes(2) / (bf_avg * 1e-3) / 1e9 / peak,
                           "traffic": NCU_TRAFFIC_BYTES["bfloat16"] if world == 1 else None},
            "clocks": clock_summary,
            "parity": parity,
            "value_broadcast_ms": bcast_ms,
        }
        if replication is not None:
            line["with_value_replication"] = replication
        if head_split is not None:
            line["head_split"] = head_split
        line["dcnv2"] = dcn_result
        if world == 1:
            line["other_msda"] = bench_other_msda(device)
        if world == 1 and not args.no_cpu_baseline:
            r = cpu_reference_throughput(workload, 15.0, 2, 1, single_thread_seconds=8.0)
            line["cpu_baseline"] = {"value": r["rate"] / 1e9, "unit": UNIT, "cores": r["cores"], "kind": r["kind"],
                                    "sample": r["sample"], "single_thread_cli_loop": r.get("single_thread")}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
