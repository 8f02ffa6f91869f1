"""vyre_b200: Blackwell (sm_100a) native backend for vyre's quantized-inference hot path.

The product is libvyre_b200.so (C ABI in include/vyre_b200.h, CUDA kernels under csrc/kernels). This package
is the thin host-side mirror of the reference's operator and submission interface used by the tests and the
benchmark; it never computes and has no fallback when the library or a device is missing.
"""
from . import ffi  # noqa: F401
from .api import *  # noqa: F401,F403
from .api import ArtifactSession, BackendError, BindingSet, Device, Program  # noqa: F401
