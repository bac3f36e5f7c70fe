from .params import (
    check_dilation_kernel_vs_input,
    check_kernel_size_vs_input,
    check_stride_vs_kernel,
    normalize_kernel_size,
    normalize_tuple_param,
)
from .window import (get_pb_start, get_pb_start_vectorized, get_window_end, get_window_start,
                     get_window_start_vectorized)

__all__ = [
    "check_dilation_kernel_vs_input", "check_kernel_size_vs_input", "check_stride_vs_kernel",
    "normalize_kernel_size", "normalize_tuple_param", "get_window_start", "get_window_end",
    "get_window_start_vectorized", "get_pb_start", "get_pb_start_vectorized",
]
