"""Architectures known to the registry; importing this package registers them."""
from . import kakipel, karorax, libulorn, lipelix, qwen2  # noqa: F401
from .kakipel import build_kakipel
from .karorax import build_karorax
from .libulorn import build_libulorn
from .lipelix import build_lipelix
from .qwen2 import build_qwen2

__all__ = ["build_kakipel", "build_karorax", "build_libulorn", "build_lipelix", "build_qwen2"]
