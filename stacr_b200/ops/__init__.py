"""Hand-written sm_100a kernels (``csrc/``) and their Python entry points."""

from ._lib import KernelError, available, check_status, lib_path, load  # noqa: F401
