"""compute_b200 — a B200 (sm_100a) backend for gomlx/compute's inference hot path.

FusedQuantizedDense, DotGeneral and FusedScaledDotProductAttention as hand-written
CUDA kernels behind a C ABI (include/cudabackend.h, libcudabackend.so).  This
package is the host-side mirror of the reference's Backend / Builder / Function /
Executable / Buffer interface over that ABI.  There is no CPU fallback: importing
works without a GPU (plans can be built), running anything needs one.
"""
from . import backend, device
from ._lib import BackendError, ErrNotImplemented, load as load_library

__all__ = ["backend", "device", "BackendError", "ErrNotImplemented", "load_library"]
