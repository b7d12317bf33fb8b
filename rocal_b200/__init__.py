"""rocal_b200 — B200 (sm_100a) implementation of rocAL's batched image-augmentation path.

Importing the package loads librocal_b200.so; there is no CPU fallback."""
from . import tables  # noqa: F401
from ._lib import LIB_PATH, Rb200Error, launch_count, version  # noqa: F401
