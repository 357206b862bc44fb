from .fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction  # noqa: F401
from .fused_linear_cross_entropy import fused_linear_cross_entropy_backward  # noqa: F401
from .fused_linear_cross_entropy import fused_linear_cross_entropy_forward  # noqa: F401
