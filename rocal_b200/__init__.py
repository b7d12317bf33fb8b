"""rocal_b200 — B200 (sm_100a) implementation of rocAL's batched image-augmentation path.

Importing the package loads librocal_b200.so; there is no CPU fallback. The one exception is the builder itself
(`python -m rocal_b200.build`), which has to be importable before the library exists."""
import sys as _sys

from . import tables  # noqa: F401

_running_builder = "rocal_b200.build" in getattr(_sys, "orig_argv", []) and "-m" in getattr(_sys, "orig_argv", [])
if not _running_builder:
    from ._lib import LIB_PATH, Rb200Error, launch_count, version  # noqa: F401
