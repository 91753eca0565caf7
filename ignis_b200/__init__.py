"""B200-native quantized linear layers behind the ignis entry points.

The package is a thin host-side mirror of the C ABI in ``include/``: device memory and streams
come from PyTorch, every computation runs in ``libignis_b200.so`` (hand-written sm_100a CUDA).
There is no CPU fallback: importing works anywhere, calling an op without the built library or
without a CUDA device raises.
"""
from . import _lib  # noqa: F401
from . import nvfp4  # noqa: F401
from . import trellis  # noqa: F401
from . import moe  # noqa: F401

__all__ = ["nvfp4", "trellis", "moe"]
