"""Hand-written sm_100a kernels (sources in ``csrc/``) and their Python wrappers."""
from . import ops  # noqa: F401
