"""B200-native INT8 W8A8 linear layer (drop-in for fish-audio-cpp's kernel boundary).

The product is the CUDA library ``lib/libw8a8.so`` (C ABI in ``include/w8a8.h``); this
package is its thin host-side binding plus the seeded synthetic workloads the tests and the
benchmark share. There is no CPU or PyTorch fallback: without the built library every call
raises.
"""
from .capi import (  # noqa: F401
    ACT_PER_TOKEN,
    ACT_PER_TOKEN_GROUP,
    EPI_NONE,
    EPI_RESIDUAL,
    EPI_SWIGLU,
    KERNEL_AUTO,
    KERNEL_GEMM,
    KERNEL_GEMM_PAIR,
    KERNEL_GEMM_SINGLE,
    KERNEL_GEMV,
    KERNEL_GEMV_PACKED,
    KERNEL_GEMV_TMA,
    KERNEL_GENERIC,
    TAIL_GROUPQUANT,
    TAIL_NONE,
    TAIL_ROWNORM,
    Context,
    W8A8Error,
    library_path,
    linear_static_scratch,
    load_library,
    num_groups,
    static_scratch_bytes,
    static_scratch_check_status,
)
