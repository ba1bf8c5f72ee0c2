"""Drop-in module named `sharq_ops`.

Point the reference's loader at this directory (SHARQ_KERNEL_BUILD=<repo>/sharq_b200/dropin,
or SHARQ_VLLM_KERNEL_BUILD for its vLLM plugin) and `sharq_loader.load_sharq_ops()` imports this
file instead of the reference's compiled extension; every op name of the reference's
extension is re-exported from sharq_b200.ops.
"""
import sys
from pathlib import Path

_ROOT = Path(__file__).resolve().parents[2]
if str(_ROOT) not in sys.path:
    sys.path.insert(0, str(_ROOT))

from sharq_b200.ops import (  # noqa: E402,F401
    compress_sparse_a,
    duplicate_sfa32_to_sfa16,
    fused_rmsnorm_sparse_residual_quantize_x,
    fused_sparse_residual_quantize_x,
    fused_sparse_residual_quantize_x_debug,
    get_fused_sparse_residual_buffer_sizes,
    get_sparse_nvfp4_buffer_sizes,
    matmul,
    matmul_accum,
    matmul_accum_tensor_scale,
    matmul_tensor_scale,
    quantize_w32_shared,
    quantize_w_nvfp4,
    quantize_x_nvfp4,
    reorder_quantize_w,
    reorder_quantize_x,
    sharq_linear_forward,
    sparse_matmul,
    sparse_matmul_tensor_scale,
)
