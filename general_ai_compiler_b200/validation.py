"""Input binding and tensor comparison, after ``src/gac/validation``.

``bind_inputs`` enforces the graph ABI on host arrays before any device work
(reference.py:14-29); ``compare_tensor`` reports the metrics the reference's
golden bundles use (golden.py:82-125): max abs / max rel error, cosine
similarity and the fraction of elements inside ``atol + rtol*|expected|``.

There is deliberately no ``reference_run`` here: the CPU evaluator is test
infrastructure and lives outside the package.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Mapping

import numpy as np

from .errors import ValidationError
from .ir import Graph


_CHUNK_BYTES = 8 << 20     # arrays above this size are checked / copied in pieces by a few host threads
_pool = None


def host_pool():
    """A small thread pool for the host-side passes over large inputs (NumPy drops the GIL inside them)."""
    global _pool
    if _pool is None:
        import os
        from concurrent.futures import ThreadPoolExecutor

        cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        _pool = ThreadPoolExecutor(max_workers=max(1, min(16, cores)))
    return _pool


def _pieces(arr: np.ndarray):
    """Flat views of at most ``_CHUNK_BYTES``, and at least two per pool thread when the array is large enough for
    that (pieces of 1 MB or more), so that a 30 MB slab keeps the whole pool busy as well."""
    flat = arr.reshape(-1)
    nbytes = min(_CHUNK_BYTES, max(1 << 20, arr.nbytes // 32))
    step = max(1, nbytes // max(1, arr.itemsize))
    return [flat[i:i + step] for i in range(0, flat.size, step)]


def all_finite(arr: np.ndarray) -> bool:
    """``np.all(np.isfinite(arr))`` for a C-contiguous array, in pieces over the host pool when it is large."""
    if arr.nbytes <= 2 * _CHUNK_BYTES:
        return bool(np.all(np.isfinite(arr)))
    return all(host_pool().map(lambda piece: bool(np.isfinite(piece).all()), _pieces(arr)))


def parallel_copy(dst: np.ndarray, src: np.ndarray) -> None:
    """``np.copyto(dst, src)`` for same-shape C-contiguous arrays, in pieces over the host pool when they are large."""
    if src.nbytes <= 2 * _CHUNK_BYTES or not (dst.flags.c_contiguous and src.flags.c_contiguous):
        np.copyto(dst, src)
        return
    list(host_pool().map(lambda pair: np.copyto(pair[0], pair[1]), zip(_pieces(dst), _pieces(src))))


_CACHE_BYTES = 512 << 10   # a piece this small is still in the core's cache when it is read a second time


def checked_copy(dst: np.ndarray, src: np.ndarray, name: str) -> None:
    """``np.copyto(dst, src)`` that also raises ``ValidationError`` when ``src`` holds a non-finite value, as ONE pass
    over memory: every piece is tested and then copied while it is still in cache, pieces spread over the host pool
    (a separate ``all_finite`` and ``parallel_copy`` read the source from memory twice).  ``dst`` is written up to
    the piece that failed."""
    if not (dst.flags.c_contiguous and src.flags.c_contiguous) or dst.shape != src.shape:
        if not all_finite(src):
            raise ValidationError(f"input {name!r} must contain finite values")
        np.copyto(dst, src)
        return
    step = max(1, _CACHE_BYTES // max(1, src.itemsize))

    def one(pair) -> bool:
        d, s = pair
        ok = True
        for i in range(0, s.size, step):
            piece = s[i:i + step]
            ok = ok and bool(np.isfinite(piece).all())
            d[i:i + step] = piece
        return ok

    pairs = list(zip(_pieces(dst), _pieces(src)))
    results = map(one, pairs) if src.nbytes <= 2 * _CHUNK_BYTES else host_pool().map(one, pairs)
    if not all(list(results)):
        raise ValidationError(f"input {name!r} must contain finite values")


def bind_inputs(graph: Graph, inputs: Mapping[str, np.ndarray], *, check_finite: bool = True) -> dict:
    """Exact names, shapes, dtypes, C-contiguity and finiteness; nothing is copied."""
    if set(inputs) != set(graph.inputs):
        raise ValidationError(f"input names must be {sorted(graph.inputs)}, got {sorted(inputs)}")
    bound = {}
    for name, spec in graph.inputs.items():
        arr = np.asarray(inputs[name])
        if arr.shape != spec.shape or arr.dtype.name != spec.dtype:
            raise ValidationError(
                f"input {name!r} requires {spec.shape}/{spec.dtype}, got {arr.shape}/{arr.dtype}")
        if not arr.flags.c_contiguous:
            raise ValidationError(f"input {name!r} must be C-contiguous")
        if check_finite and not all_finite(arr):
            raise ValidationError(f"input {name!r} must contain finite values")
        bound[name] = arr
    return bound


@dataclass(frozen=True)
class TensorTolerance:
    """The fp32 gate of this path: |a-b| <= 1e-4 + 1e-5*|b| everywhere."""

    rtol: float = 1e-5
    atol: float = 1e-4
    cosine_min: float = 0.99999


@dataclass(frozen=True)
class TensorComparison:
    shape: tuple
    dtype: str
    max_abs: float
    max_rel: float
    cosine: float
    close_fraction: float
    passed: bool

    def to_dict(self) -> dict:
        return asdict(self)


def compare_tensor(actual, expected, tolerance: TensorTolerance | None = None) -> TensorComparison:
    tol = tolerance or TensorTolerance()
    a, e = np.asarray(actual), np.asarray(expected)
    if a.shape != e.shape:
        raise ValidationError(f"golden shape mismatch: actual {a.shape}, expected {e.shape}")
    if not np.issubdtype(a.dtype, np.number) or not np.issubdtype(e.dtype, np.number):
        raise ValidationError("golden comparison requires numeric arrays")
    if not np.all(np.isfinite(a)) or not np.all(np.isfinite(e)):
        raise ValidationError("golden comparison requires finite arrays")
    x = a.astype(np.float64).reshape(-1)
    y = e.astype(np.float64).reshape(-1)
    if x.size == 0:
        return TensorComparison(tuple(a.shape), a.dtype.name, 0.0, 0.0, 1.0, 1.0, True)
    diff = np.abs(x - y)
    nx, ny = float(np.linalg.norm(x)), float(np.linalg.norm(y))
    if nx == 0.0 and ny == 0.0:
        cosine = 1.0
    elif nx == 0.0 or ny == 0.0:
        cosine = 0.0
    else:
        cosine = float(np.clip(np.dot(x, y) / (nx * ny), -1.0, 1.0))
    close = float(np.mean(diff <= tol.atol + tol.rtol * np.abs(y)))
    return TensorComparison(tuple(a.shape), a.dtype.name, float(diff.max()),
                            float((diff / np.maximum(np.abs(y), np.finfo(np.float64).tiny)).max()), cosine, close,
                            close == 1.0 and cosine >= tol.cosine_min)
