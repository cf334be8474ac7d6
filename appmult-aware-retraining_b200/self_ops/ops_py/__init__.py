from .approx_ops import (
    init_lookup_tables,
    set_lookup_tables,
    approx_gemm_op,
    approx_gemm_baseline_op,
    approx_conv2d_op,
    approx_conv2d_baseline_op,
    approx_conv2d_fused_op,
    approx_conv2d_fused_baseline_op,
    unfold_conv2d,
)

# the first five names are the reference's public API (self_ops/ops_py/__init__.py:1-12)
__all__ = [
    "init_lookup_tables",
    "approx_gemm_op",
    "approx_gemm_baseline_op",
    "approx_conv2d_op",
    "approx_conv2d_baseline_op",
    "set_lookup_tables",
    "approx_conv2d_fused_op",
    "approx_conv2d_fused_baseline_op",
    "unfold_conv2d",
]
