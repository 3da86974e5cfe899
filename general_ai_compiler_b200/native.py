"""ctypes binding of ``libgacb.so`` -- the only door to the CUDA kernels.

Every function here raises when the library is absent or a call fails; there
is no CPU path behind it (the reference's session makes the same promise:
``src/gac/execution/cuda.py:132-138``).
"""

from __future__ import annotations

import ctypes
from pathlib import Path

from .errors import BackendError, DeviceUnavailableError, EvaluationError

LIB_PATH = Path(__file__).resolve().parent / "libgacb.so"

GACB_OK = 0
GACB_ERR_INVALID_ARGUMENT = -1
GACB_ERR_SHAPE_MISMATCH = -2
GACB_ERR_UNSUPPORTED = -3
GACB_ERR_CUDA = -4
GACB_ERR_NO_DEVICE = -5
GACB_ERR_DEVICE_TIMEOUT = -6

GACB_F32 = 0
GACB_BF16 = 1

DCN_F32X3 = 0
DCN_TF32 = 1
DCN_BF16 = 2
DCN_REUSE_WEIGHTS = 0x100   # GACB_DCN_REUSE_WEIGHTS
DCN_REUSE_INPUT = 0x200     # GACB_DCN_REUSE_INPUT
DCN_INPUT_AT_END = 0x800    # GACB_DCN_INPUT_AT_END
DCN_MATH_MODES = {"f32x3": DCN_F32X3, "tf32": DCN_TF32, "bf16": DCN_BF16}
DCN_TEST_DROP_WEIGHT_COPIES = 0x400   # fault-injection build only (-DGACB_DCN_FAULT_INJECT=1)

_vp = ctypes.c_void_p
_i = ctypes.c_int
_sz = ctypes.c_size_t
_ip = ctypes.POINTER(ctypes.c_int32)

_fp = ctypes.c_void_p


class MsdaDesc(ctypes.Structure):
    """``gacb_msda_desc`` of include/gacb.h (field order and types must match)."""

    _fields_ = [
        ("value", _vp), ("value_dtype", _i),
        ("locations", _fp), ("attention", _fp), ("normalizer", _fp), ("reference", _fp), ("visibility", _fp),
        ("out", _fp), ("reduce_out", _fp),
        ("spatial_hw", _ip), ("norm_shape", _ip), ("coord_shape", _ip), ("ref_shape", _ip),
        ("L", _i), ("B", _i), ("S", _i), ("Q", _i), ("H", _i), ("D", _i), ("P", _i),
        ("coord_rank", _i), ("reference_first", _i), ("attention_is_logits", _i),
        ("group", _i), ("reduce_mode", _i),
        ("q_begin", _i), ("q_end", _i),
        ("compact_scratch", _vp), ("compact_scratch_bytes", _sz),
    ]


class LaunchGeometry(ctypes.Structure):
    """``gacb_launch_geometry`` of include/gacb.h."""

    _fields_ = [("grid", _i * 3), ("block", _i * 3), ("dynamic_smem_bytes", _sz), ("units_per_cta", _i),
                ("kernel", ctypes.c_char * 64)]


# name -> (restype, argtypes); must list every symbol include/gacb.h declares.
SIGNATURES = {
    "gacb_version": (_i, []),
    "gacb_last_error_string": (ctypes.c_char_p, []),
    "gacb_device_count": (_i, []),
    "gacb_device_capability": (_i, [_i]),
    "gacb_msda_forward": (_i, [_vp, _i, _vp, _vp, _vp, _ip] + [_i] * 9 + [_vp]),
    "gacb_msda_offsets_forward": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _ip] + [_i] * 7 + [_ip, _ip, _ip, _i, _i, _i, _i, _vp]),
    "gacb_msda_logits_forward": (_i, [_vp, _i, _vp, _vp, _vp, _ip] + [_i] * 9 + [_vp]),
    "gacb_msda_offsets_logits_forward": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _ip] + [_i] * 7 + [_ip, _ip, _ip, _i, _i, _i, _i, _vp]),
    "gacb_msda_run": (_i, [ctypes.POINTER(MsdaDesc), _vp]),
    "gacb_msda_tile_path": (_i, [_i]),
    "gacb_conv_window_path": (_i, [_i]),
    "gacb_dcnv2_forward": (_i, [_vp] * 6 + [_i] * 18 + [_vp, _sz, _vp, _vp]),
    "gacb_conv2d_forward": (_i, [_vp, _vp, _vp, _i, _vp, _vp] + [_i] * 20 + [_vp, _sz, _vp, _vp]),
    "gacb_conv2d_workspace_bytes": (_sz, [_i] * 17),
    "gacb_dcnv2_pixels_forward": (_i, [_vp] * 6 + [_i] * 15 + [ctypes.c_longlong] * 2 + [_i, _vp, _sz, _vp, _vp]),
    "gacb_dcnv2_rows_forward": (_i, [_vp] * 6 + [_i] * 20 + [_vp, _sz, _vp, _vp]),
    "gacb_dcnv2_fused_forward": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_float, _i, _vp]
                                 + [_i] * 18 + [_vp, _sz, _vp, _vp]),
    "gacb_dcnv2_workspace_bytes": (_sz, [_i] * 16),
    "gacb_dcnv2_forward_static": (_i, [_vp] * 6 + [_i] * 18 + [_vp, _vp]),
    "gacb_dcnv2_workspace_parts": (_i, [_i] * 19 + [ctypes.POINTER(_sz), ctypes.POINTER(_sz)]),
    "gacb_msda_launch_geometry": (_i, [_i, _ip] + [_i] * 9 + [ctypes.POINTER(LaunchGeometry)]),
    "gacb_dcnv2_launch_geometry": (_i, [_i] * 18 + [ctypes.POINTER(LaunchGeometry)]),
    "gacb_checked_violations": (_i, [ctypes.POINTER(ctypes.c_uint), ctypes.POINTER(ctypes.c_uint)]),
    "gacb_status_from_word": (_i, [ctypes.c_int32]),
    "gacb_read_status_word": (_i, [_vp, _vp]),
    "gacb_ipc_alloc": (_i, [_sz, ctypes.POINTER(_vp), ctypes.c_char_p]),
    "gacb_ipc_open": (_i, [ctypes.c_char_p, ctypes.POINTER(_vp)]),
    "gacb_ipc_close": (_i, [_vp]),
    "gacb_ipc_free": (_i, [_vp]),
    "gacb_copy_async": (_i, [_vp, _vp, _sz, _vp]),
    "gacb_peer_barrier": (_i, [ctypes.POINTER(_vp), _vp, _vp, _i, _i, _vp, _vp]),
    "gacb_cast_f32_to_bf16": (_i, [_vp, _vp, _sz, _vp]),
    "gacb_gather_probe": (_i, [_vp, _sz, _i, _i, _i, ctypes.c_uint32, _vp, ctypes.POINTER(_sz), _vp]),
}

_lib = None
CHECKED_LIB_PATH = LIB_PATH.with_name("libgacb_checked.so")          # -DGACB_CHECKED=1
FAULT_LIB_PATH = LIB_PATH.with_name("libgacb_faultinject.so")        # -DGACB_DCN_FAULT_INJECT=1, short spin limit


def load() -> ctypes.CDLL:
    """Load the library once; a missing or stale build is a hard error."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise DeviceUnavailableError(
            f"{LIB_PATH} is missing: build it with `python -m general_ai_compiler_b200.build`. "
            "There is no CPU fallback."
        )
    try:
        lib = ctypes.CDLL(str(LIB_PATH))
    except OSError as exc:
        raise DeviceUnavailableError(f"cannot load {LIB_PATH}: {exc}. There is no CPU fallback.") from exc
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise DeviceUnavailableError(f"{LIB_PATH} does not export {name}; rebuild it") from exc
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    text = load().gacb_last_error_string()
    return text.decode("utf-8", "replace") if text else ""


def check(status: int, what: str) -> None:
    """Map a gacb_status to the host error taxonomy."""
    if status == GACB_OK:
        return
    message = f"{what}: {last_error()} (gacb status {status})"
    if status in (GACB_ERR_INVALID_ARGUMENT, GACB_ERR_SHAPE_MISMATCH):
        raise EvaluationError(message)
    if status == GACB_ERR_NO_DEVICE:
        raise DeviceUnavailableError(message)
    raise BackendError(message)


def int32_table(values) -> ctypes.Array:
    flat = [int(v) for v in values]
    return (ctypes.c_int32 * len(flat))(*flat)


def msda_launch_geometry(value_dtype: int, spatial_shapes, B: int, Q: int, H: int, D: int, P: int,
                         q_range=None) -> LaunchGeometry:
    shapes = [(int(h), int(w)) for h, w in spatial_shapes]
    geo = LaunchGeometry()
    q0, q1 = (0, Q) if q_range is None else q_range
    rc = load().gacb_msda_launch_geometry(value_dtype, int32_table(v for pair in shapes for v in pair), len(shapes), B,
                                          sum(h * w for h, w in shapes), Q, H, D, P, q0, q1, ctypes.byref(geo))
    check(rc, "gacb_msda_launch_geometry")
    return geo


def dcnv2_launch_geometry(n, Cin, H, W, Cout, Kh, Kw, stride, padding, dilation, groups, deform_groups, math_mode: int,
                          plain: bool = False, sm_count: int = 0) -> LaunchGeometry:
    geo = LaunchGeometry()
    rc = load().gacb_dcnv2_launch_geometry(n, Cin, H, W, Cout, Kh, Kw, stride[0], stride[1], padding[0], padding[1],
                                           dilation[0], dilation[1], groups, deform_groups, math_mode, 1 if plain else 0,
                                           sm_count, ctypes.byref(geo))
    check(rc, "gacb_dcnv2_launch_geometry")
    return geo


def _bind(lib: ctypes.CDLL, path) -> ctypes.CDLL:
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise DeviceUnavailableError(f"{path} does not export {name}; rebuild it") from exc
        fn.restype = res
        fn.argtypes = args
    return lib


class use_library:
    """Context manager that routes every call of this module (and so of ``ops`` and ``CudaSession``) through
    another build of the library -- the checked build or the fault-injection build -- and restores the normal one
    afterwards.  For tests; not thread-safe."""

    _cache: dict = {}

    def __init__(self, path) -> None:
        self.path = str(path)

    def __enter__(self) -> ctypes.CDLL:
        global _lib
        load()
        if self.path not in self._cache:
            try:
                self._cache[self.path] = _bind(ctypes.CDLL(self.path), self.path)
            except OSError as exc:
                raise DeviceUnavailableError(f"cannot load {self.path}: {exc}") from exc
        self._previous = _lib
        _lib = self._cache[self.path]
        return _lib

    def __exit__(self, *_):
        global _lib
        _lib = self._previous
