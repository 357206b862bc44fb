from .fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction  # noqa: F401
from .fused_linear_cross_entropy import fused_linear_cross_entropy_backward  # noqa: F401
from .fused_linear_cross_entropy import fused_linear_cross_entropy_forward  # noqa: F401
from .cross_entropy import LigerCrossEntropyFunction  # noqa: F401
from .cross_entropy import cross_entropy_backward  # noqa: F401
from .cross_entropy import cross_entropy_forward  # noqa: F401
