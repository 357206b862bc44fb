"""B200-native fused linear cross-entropy with the call surface of Liger-Kernel's FLCE path.

Importing this package loads ``libflce_b200.so``; if it has not been built the import fails
(there is no fallback implementation).
"""

from . import _lib  # noqa: F401  (loads the shared library, raises if missing)
from .ops.cross_entropy import LigerCrossEntropyFunction  # noqa: F401
from .ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction  # noqa: F401
from .ops.fused_linear_jsd import LigerFusedLinearJSDFunction  # noqa: F401
from .ops.fused_linear_scaled_cross_entropy import LigerFusedLinearScaledCrossEntropyFunction  # noqa: F401
from .ops.fused_rmsnorm_linear_cross_entropy import LigerFusedRMSNormLinearCrossEntropyFunction  # noqa: F401
from .ops.fused_rmsnorm_linear_cross_entropy import liger_fused_rmsnorm_linear_cross_entropy  # noqa: F401
from .transformers.cross_entropy import LigerCrossEntropyLoss  # noqa: F401
from .transformers.functional import liger_cross_entropy  # noqa: F401
from .transformers.functional import CrossEntropyOutput  # noqa: F401
from .transformers.functional import liger_fused_linear_cross_entropy  # noqa: F401
from .transformers.functional import liger_fused_linear_jsd  # noqa: F401
from .transformers.fused_linear_jsd import LigerFusedLinearJSD  # noqa: F401
from .transformers.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyLoss  # noqa: F401
from .transformers.model.loss_utils import LigerForCausalLMLoss  # noqa: F401
from .transformers.monkey_patch import _apply_liger_kernel_to_instance  # noqa: F401
from .transformers.monkey_patch import MODEL_TYPE_TO_APPLY_LIGER_FN  # noqa: F401
from .transformers.monkey_patch import *  # noqa: F401,F403  (apply_liger_kernel_to_<family>, one per family in monkey_patch._FAMILIES)
from .transformers.monkey_patch import install  # noqa: F401

__version__ = "0.1.0"
