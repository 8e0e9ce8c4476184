"""mixedgemm_b200: B200 (sm_100a) implementation of MixedGemm's hot path - activation /
weight reorder-and-quantise into MXFP4 / MXFP6 / MXFP8 and the mixed block-scaled GEMM -
behind the reference's Python entry points and a C ABI (include/mixedgemm_c.h)."""
from .api import (ShardedActivation, alloc_quantized_w, alloc_quantized_x, device_status, matmul, matmul_group, matmul_multi,  # noqa: F401
                  reorder_index, reorder_quantize_w, reorder_quantize_x, reorder_quantize_x_multi, reset_options, set_option, set_wait_limit_us,
                  sf_bytes, test_function)

__all__ = ["ShardedActivation", "matmul", "matmul_group", "matmul_multi", "reorder_quantize_x_multi", "reorder_index", "reorder_quantize_x", "reorder_quantize_w",
           "test_function", "sf_bytes", "device_status", "set_option", "reset_options", "set_wait_limit_us"]
