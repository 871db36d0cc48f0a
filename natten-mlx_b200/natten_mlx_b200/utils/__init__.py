from .params import (check_dilation_kernel_vs_input, check_kernel_size_vs_input, check_stride_vs_kernel,
                     normalize_kernel_size, normalize_tuple_param)
from .window import (compute_pb_start, compute_window_start_end, get_pb_start, get_window_end,
                     get_window_start)

__all__ = [
    "check_dilation_kernel_vs_input", "check_kernel_size_vs_input", "check_stride_vs_kernel",
    "normalize_kernel_size", "normalize_tuple_param", "compute_pb_start", "compute_window_start_end",
    "get_pb_start", "get_window_end", "get_window_start",
]
