"""B200-native kernels for the MOD-DiT sparse-attention path (ctypes binding + tensor-level ops)."""
from . import _lib  # noqa: F401  (raises if the shared library is missing)
from . import ops  # noqa: F401

__all__ = ["ops"]
