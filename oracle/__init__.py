"""CPU oracles for the deformable-sampling path -- TEST INFRASTRUCTURE ONLY.

Nothing under ``oracle/`` is part of the shipped package.  It may be imported
by ``tests/``, by the smoke check and by the CPU-baseline / reference legs of
the benchmark, and only as the checker or as the CPU arm being timed.

``msda_numpy``   NumPy restatement of src/gac/core/ops.py:787-851 (pinned
                 bit-for-bit to the real evaluator by tests/golden/make_golden.py).
``gac_oracle.c`` C restatement of the same MSDA arithmetic and of the native
                 DCNv2 lowering (native/lib/DeviceLowering.cpp:605-698,
                 :251-286); loaded through :func:`load_c_oracle`.
``_ref/``        (never committed) the reference's own evaluator modules, placed
                 there by ``make_ref.py`` from a checkout; :func:`load_reference`
                 imports them.  Used as the timed CPU arm (kind "reference") and
                 to re-check the restatements wherever the directory exists.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libgac_oracle.so"
_lib = None


def build_c_oracle(force: bool = False) -> Path:
    """Compile ``gac_oracle.c`` with the committed Makefile (gcc only)."""
    src = _HERE / "gac_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "libgac_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def load_c_oracle():
    global _lib
    if _lib is None:
        build_c_oracle()
        lib = ctypes.CDLL(str(_LIB_PATH))
        fp = ctypes.POINTER(ctypes.c_float)
        ip = ctypes.POINTER(ctypes.c_int32)
        lib.gac_oracle_msda_f32.restype = ctypes.c_int
        lib.gac_oracle_msda_f32.argtypes = [fp, fp, fp, fp, ip] + [ctypes.c_int] * 8
        lib.gac_oracle_dcnv2_f32.restype = ctypes.c_int
        lib.gac_oracle_dcnv2_f32.argtypes = [fp] * 6 + [ctypes.c_int] * 16
        lib.gac_oracle_conv2d_f32.restype = ctypes.c_int
        lib.gac_oracle_conv2d_f32.argtypes = [fp] * 4 + [ctypes.c_int] * 18
        _lib = lib
    return _lib


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def msda_c(value, locations, weights, spatial_shapes, threads: int = 0) -> np.ndarray:
    """MSDA through the C oracle; same layouts as :func:`oracle.msda_numpy.msda_forward`."""
    lib = load_c_oracle()
    value, pv = _f32(value)
    locations, pl = _f32(locations)
    weights, pw = _f32(weights)
    B, S, H, D = value.shape
    Q, L, P = locations.shape[1], locations.shape[3], locations.shape[4]
    hw = np.ascontiguousarray(np.asarray(spatial_shapes, dtype=np.int32).reshape(-1))
    if hw.size != 2 * L:
        raise ValueError("spatial_shapes must hold one [H, W] pair per level")
    out = np.empty((B, Q, H * D), np.float32)
    rc = lib.gac_oracle_msda_f32(pv, pl, pw, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                                 hw.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)),
                                 L, B, S, Q, H, D, P, int(threads))
    if rc != 0:
        raise ValueError(f"gac_oracle_msda_f32 rejected the shapes (code {rc})")
    return out


def dcnv2_c(x, offset, mask, weight, bias=None, *, stride=(1, 1), padding=(0, 0),
            dilation=(1, 1), groups=1, deform_groups=1, threads: int = 0) -> np.ndarray:
    """DCNv2 through the C oracle: X NCHW, offset (dy,dx interleaved), mask, W OIHW."""
    lib = load_c_oracle()
    x, px = _f32(x)
    offset, po = _f32(offset)
    mask, pm = _f32(mask)
    weight, pw = _f32(weight)
    N, Cin, H, W = x.shape
    Cout, _, Kh, Kw = weight.shape
    Ho = (H + 2 * padding[0] - dilation[0] * (Kh - 1) - 1) // stride[0] + 1
    Wo = (W + 2 * padding[1] - dilation[1] * (Kw - 1) - 1) // stride[1] + 1
    y = np.empty((N, Cout, Ho, Wo), np.float32)
    if bias is not None:
        bias, pb = _f32(bias)
    else:
        pb = ctypes.POINTER(ctypes.c_float)()
    rc = lib.gac_oracle_dcnv2_f32(px, po, pm, pw, pb, y.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                                  N, Cin, H, W, Cout, Kh, Kw, stride[0], stride[1], padding[0],
                                  padding[1], dilation[0], dilation[1], groups, deform_groups,
                                  int(threads))
    if rc != 0:
        raise ValueError(f"gac_oracle_dcnv2_f32 rejected the configuration (code {rc})")
    return y


def conv2d_c(x, weight, bias=None, *, strides=(1, 1), pads=(0, 0, 0, 0), dilations=(1, 1), groups=1,
             relu: bool = False, threads: int = 0) -> np.ndarray:
    """Plain convolution through the C oracle: X NCHW, W OIHW, pads (top, left, bottom, right)."""
    lib = load_c_oracle()
    x, px = _f32(x)
    weight, pw = _f32(weight)
    N, Cin, H, W = x.shape
    Cout, _, Kh, Kw = weight.shape
    Ho = (H + pads[0] + pads[2] - dilations[0] * (Kh - 1) - 1) // strides[0] + 1
    Wo = (W + pads[1] + pads[3] - dilations[1] * (Kw - 1) - 1) // strides[1] + 1
    y = np.empty((N, Cout, Ho, Wo), np.float32)
    if bias is not None:
        bias, pb = _f32(bias)
    else:
        pb = ctypes.POINTER(ctypes.c_float)()
    rc = lib.gac_oracle_conv2d_f32(px, pw, pb, y.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), N, Cin, H, W,
                                   Cout, Kh, Kw, strides[0], strides[1], pads[0], pads[1], pads[2], pads[3],
                                   dilations[0], dilations[1], groups, 1 if relu else 0, int(threads))
    if rc != 0:
        raise ValueError(f"gac_oracle_conv2d_f32 rejected the configuration (code {rc})")
    return y


def sigmoid_ref(x: np.ndarray) -> np.ndarray:
    """The reference's Sigmoid op, stable form (src/gac/core/ops.py:916-924)."""
    x = np.asarray(x, np.float32)
    out = np.empty_like(x)
    pos = x >= 0
    out[pos] = 1 / (1 + np.exp(-x[pos]))
    e = np.exp(x[~pos])
    out[~pos] = e / (1 + e)
    return out


def dcnv2_fused_c(x, offset, mask_logits, weight, bias, bn=None, relu=False, **conv) -> np.ndarray:
    """Sigmoid -> DCNv2 -> BatchNorm ((v-mean)/sqrt(var+eps)*scale+bias, src/gac/core/ops.py:1084-1089) -> ReLU,
    each step as the reference evaluates the separate ops."""
    y = dcnv2_c(x, offset, sigmoid_ref(mask_logits), weight, bias, **conv)
    if bn is not None:
        scale, b, mean, var, eps = bn
        shp = (1, -1, 1, 1)
        y = ((y - mean.reshape(shp)) / np.sqrt(var.reshape(shp) + np.float32(eps)) * scale.reshape(shp)
             + b.reshape(shp)).astype(np.float32)
    if relu:
        y = np.maximum(y, np.float32(0))
    return y


def host_threads() -> int:
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


_REF_DIR = _HERE / "_ref"
_reference = None


def reference_available() -> bool:
    return (_REF_DIR / "gac" / "core" / "ops.py").is_file()


def load_reference():
    """The reference's own modules from ``oracle/_ref`` (see ``make_ref.py``) as a namespace with ``evaluate_op``,
    ``reference_run``, ``Graph``, ``Node`` and ``TensorSpec``; raises ``FileNotFoundError`` when they are absent."""
    global _reference
    if _reference is None:
        if not reference_available():
            raise FileNotFoundError(f"{_REF_DIR} is empty: run oracle/make_ref.py on a box that has the reference checkout")
        import importlib
        import sys
        from types import SimpleNamespace

        sys.dont_write_bytecode = True
        sys.path.insert(0, str(_REF_DIR))
        try:
            ops = importlib.import_module("gac.core.ops")
            ir = importlib.import_module("gac.core.ir")
            ref = importlib.import_module("gac.validation.reference")
        finally:
            sys.path.remove(str(_REF_DIR))
        _reference = SimpleNamespace(evaluate_op=ops.evaluate_op, reference_run=ref.reference_run, Graph=ir.Graph,
                                     Node=ir.Node, TensorSpec=ir.TensorSpec)
    return _reference


def reference_msda_graph(ref, batch, spatial_size, queries, heads, head_dim, levels, points, spatial_shapes):
    """The one-node MSDA graph in the reference's own IR (node recipe of its tests/test_bevformer_msda.py:23-30)."""
    spec = ref.TensorSpec
    inputs = {"value": spec((batch, spatial_size, heads, head_dim), "float32"),
              "sampling_locations": spec((batch, queries, heads, levels, points, 2), "float32"),
              "attention_weights": spec((batch, queries, heads, levels, points), "float32")}
    node = ref.Node("msda", "MSDeformableAttention", ("value", "sampling_locations", "attention_weights"), ("output",),
                    {"spatial_shapes": [list(map(int, s)) for s in spatial_shapes]})
    return ref.Graph("msda", inputs, ("output",), [node])
