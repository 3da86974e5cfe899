"""Failure reporting that needs no GPU: status word -> error code -> ``BackendError`` + invalid session, and
argument combinations the library must refuse before it enqueues anything.

The reference marks a session failed after any device-side failure and refuses further runs
(src/gac/execution/cuda.py:457-464); its native runner reports ``status: "failed"`` with the failing stage
(native/runtime/cuda-run.cpp:685-703).  Here a kernel whose bounded wait ran out sets a device status word; these
tests inject that word on the host.
"""

from __future__ import annotations

import ctypes
from threading import Lock

import pytest

from general_ai_compiler_b200 import native
from general_ai_compiler_b200.errors import BackendError, EvaluationError
from general_ai_compiler_b200.session import CudaSession


def test_status_word_maps_to_device_timeout():
    lib = native.load()
    assert lib.gacb_status_from_word(0) == native.GACB_OK
    assert lib.gacb_status_from_word(1) == native.GACB_ERR_DEVICE_TIMEOUT
    assert "bounded wait" in native.last_error()
    with pytest.raises(BackendError, match="bounded wait"):
        native.check(lib.gacb_status_from_word(7), "device status word")


def test_set_status_word_invalidates_the_session():
    session = CudaSession.__new__(CudaSession)        # no device: only the failure bookkeeping is exercised
    session._failed, session._closed, session._lock = False, False, Lock()
    session._check_device_status(word=0)
    assert session._failed is False
    with pytest.raises(BackendError, match="bounded wait"):
        session._check_device_status(word=1)
    assert session._failed is True
    with pytest.raises(BackendError, match="closed or failed"):
        session.run({})
    with pytest.raises(BackendError, match="closed or failed"):
        session.run_resident(1)


def test_mean_reduction_refuses_a_visibility_tensor():
    """Rows masked out by visibility are never written, and the plain mean would read them."""
    lib = native.load()
    desc = native.MsdaDesc()
    fake = 0x1000      # never dereferenced: the call is refused while it checks its arguments
    table = native.int32_table([2, 3])
    desc.value, desc.locations, desc.attention, desc.out, desc.reduce_out, desc.visibility = (fake,) * 6
    desc.spatial_hw = table
    desc.L, desc.B, desc.S, desc.Q, desc.H, desc.D, desc.P = 1, 2, 6, 4, 2, 8, 4
    desc.group, desc.reduce_mode, desc.q_begin, desc.q_end = 2, 2, 0, 4
    assert lib.gacb_msda_run(ctypes.byref(desc), None) == native.GACB_ERR_INVALID_ARGUMENT
    assert "visibility" in native.last_error()
    with pytest.raises(EvaluationError):
        native.check(native.GACB_ERR_INVALID_ARGUMENT, "gacb_msda_run")
    # a bad descriptor is refused before the compaction pass is enqueued as well
    desc.reduce_mode, desc.S = 1, 7
    desc.compact_scratch, desc.compact_scratch_bytes = fake, 1 << 20
    assert lib.gacb_msda_run(ctypes.byref(desc), None) == native.GACB_ERR_SHAPE_MISMATCH
