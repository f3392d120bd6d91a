"""e_natten_b200: fused neighborhood attention for NVIDIA B200, drop-in for
``e_natten.natten2d`` / ``e_natten.natten1d`` (e_natten/__init__.py:1).  Importing fails if
libna2d.so is not built."""
from .functional import (  # noqa: F401
    Natten1d,
    Natten2d,
    as_kernel_input,
    check_kernels,
    device_index_tables,
    get_backward_window_end,
    get_backward_window_start,
    get_window_start,
    launch_count,
    make_rows,
    natten1d,
    natten1d_backward,
    natten1d_forward,
    natten2d,
    natten2d_backward,
    natten2d_forward,
    natten2d_unfused,
    natten2d_with_lse,
    natten2dav,
    natten2dqk,
    poll_kernels,
)

__all__ = [
    "natten2d", "natten2d_with_lse", "natten2d_forward", "natten2d_backward", "Natten2d", "make_rows",
    "natten1d", "natten1d_forward", "natten1d_backward", "Natten1d",
    "natten2dqk", "natten2dav", "natten2d_unfused",
    "get_window_start", "get_backward_window_start", "get_backward_window_end",
    "device_index_tables", "check_kernels", "poll_kernels", "launch_count", "as_kernel_input",
]
