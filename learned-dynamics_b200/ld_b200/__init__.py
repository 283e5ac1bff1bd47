"""B200-native kernels for the equivariant message-passing hot path of learned-dynamics."""
from . import _lib  # noqa: F401
