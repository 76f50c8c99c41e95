"""neus2_b200: Blackwell-native (sm_100a) kernels for the NeuS2 training step, behind the C ABI of include/neus2b.h.

`neus2_b200.ops` exposes each C entry point on torch CUDA tensors; the CUDA shared library is the only compute path."""
from . import _lib  # noqa: F401

__all__ = ["_lib", "ops"]
