"""Error taxonomy of the host API.

Same class names and inheritance as GAC's ``src/gac/core/errors.py:6-35`` so
that callers and tests written against the reference catch the same types.
"""

from __future__ import annotations


class GACError(Exception):
    """Root of every expected, user-facing failure."""


class ValidationError(GACError):
    """An IR object or a bound input breaks a structural rule (raised before any device work)."""


class ShapeInferenceError(GACError):
    """An operator's output shape/dtype cannot be derived from its inputs."""


class EvaluationError(GACError):
    """An operator evaluator was handed tensors that violate its contract."""


class PassError(GACError):
    """A graph pass (``passes.fuse_deformable_sampling``) met a sub-graph it cannot rewrite consistently."""


class BackendError(GACError):
    """The B200 backend cannot compile or execute the requested program."""


class DeviceUnavailableError(BackendError):
    """No usable sm_100 device, or the native library is missing.  Never followed by a CPU fallback."""
