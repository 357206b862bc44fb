from .cross_entropy import LigerCrossEntropyLoss  # noqa: F401
from .functional import CrossEntropyOutput  # noqa: F401
from .functional import liger_cross_entropy  # noqa: F401
from .functional import liger_fused_linear_cross_entropy  # noqa: F401
from .functional import liger_fused_linear_jsd  # noqa: F401
from .fused_linear_jsd import LigerFusedLinearJSD  # noqa: F401
from .fused_linear_cross_entropy import LigerFusedLinearCrossEntropyLoss  # noqa: F401
from .monkey_patch import _apply_liger_kernel_to_instance  # noqa: F401
from .monkey_patch import MODEL_TYPE_TO_APPLY_LIGER_FN  # noqa: F401
from .monkey_patch import *  # noqa: F401,F403  (apply_liger_kernel_to_<family>, one per family in monkey_patch._FAMILIES)
