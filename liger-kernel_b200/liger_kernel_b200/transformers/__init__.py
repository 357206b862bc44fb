from .functional import CrossEntropyOutput  # noqa: F401
from .functional import liger_fused_linear_cross_entropy  # noqa: F401
from .fused_linear_cross_entropy import LigerFusedLinearCrossEntropyLoss  # noqa: F401
from .monkey_patch import _apply_liger_kernel_to_instance  # noqa: F401
from .monkey_patch import apply_liger_kernel_to_gemma2  # noqa: F401
from .monkey_patch import apply_liger_kernel_to_llama  # noqa: F401
from .monkey_patch import apply_liger_kernel_to_qwen2  # noqa: F401
