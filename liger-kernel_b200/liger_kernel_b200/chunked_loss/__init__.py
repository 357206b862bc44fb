"""Preference losses (``preference.py``), GRPO (``grpo.py``) and JSD distillation (``distillation.py``) of the reference's ``liger_kernel.chunked_loss`` on this
library's fused head."""

from .distillation import LigerFusedLinearCosineSimilarityFunction  # noqa: F401
from .distillation import LigerFusedLinearCosineSimilarityLoss  # noqa: F401
from .distillation import LigerFusedLinearJSDFunction  # noqa: F401
from .distillation import LigerFusedLinearJSDLoss  # noqa: F401
from .grpo import LigerFusedLinearGRPOFunction  # noqa: F401
from .grpo import LigerFusedLinearGRPOLoss  # noqa: F401
from .grpo import selected_token_logps  # noqa: F401
from .preference import LigerFusedLinearCPOFunction  # noqa: F401
from .preference import LigerFusedLinearCPOLoss  # noqa: F401
from .preference import LigerFusedLinearDPOFunction  # noqa: F401
from .preference import LigerFusedLinearDPOLoss  # noqa: F401
from .preference import LigerFusedLinearKTOFunction  # noqa: F401
from .preference import LigerFusedLinearKTOLoss  # noqa: F401
from .preference import LigerFusedLinearORPOFunction  # noqa: F401
from .preference import LigerFusedLinearORPOLoss  # noqa: F401
from .preference import LigerFusedLinearSimPOFunction  # noqa: F401
from .preference import LigerFusedLinearSimPOLoss  # noqa: F401
from .preference import per_token_logps  # noqa: F401

liger_fused_linear_dpo = LigerFusedLinearDPOFunction.apply
liger_fused_linear_orpo = LigerFusedLinearORPOFunction.apply
liger_fused_linear_simpo = LigerFusedLinearSimPOFunction.apply
liger_fused_linear_cpo = LigerFusedLinearCPOFunction.apply
liger_fused_linear_kto = LigerFusedLinearKTOFunction.apply
liger_fused_linear_grpo = LigerFusedLinearGRPOFunction.apply
liger_fused_linear_jsd = LigerFusedLinearJSDFunction.apply
liger_fused_linear_cosine = LigerFusedLinearCosineSimilarityFunction.apply
