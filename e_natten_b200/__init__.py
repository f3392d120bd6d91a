"""e_natten_b200: fused 2D neighborhood attention for NVIDIA B200, drop-in for
``e_natten.natten2d`` (e_natten/__init__.py:1).  Importing fails if libna2d.so is not built."""
from .functional import (  # noqa: F401
    Natten2d,
    check_kernels,
    device_index_tables,
    get_backward_window_end,
    get_backward_window_start,
    get_window_start,
    launch_count,
    make_rows,
    natten2d,
    natten2d_backward,
    natten2d_forward,
    natten2d_with_lse,
)

__all__ = [
    "natten2d", "natten2d_with_lse", "natten2d_forward", "natten2d_backward", "Natten2d", "make_rows",
    "get_window_start", "get_backward_window_start", "get_backward_window_end",
    "device_index_tables", "check_kernels", "launch_count",
]
