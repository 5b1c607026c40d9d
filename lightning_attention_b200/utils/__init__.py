from .utils import _build_slope_tensor, get_memory  # noqa: F401

__all__ = ["_build_slope_tensor", "get_memory"]
