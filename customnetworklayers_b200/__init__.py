"""B200-native optimisation layers: the unrolled FISTA TV-inpainting layer with its hand-derived backward pass,
as hand-written sm_100a CUDA behind the reference's Python layer API.  CUDA only; there is no CPU fallback."""
from . import _lib  # noqa: F401
from .TVInpainting import TVInpaint, TVInpaintingFunction  # noqa: F401

__all__ = ["TVInpaint", "TVInpaintingFunction"]
