"""``LigerFusedLinearJSD`` module, constructor- and call-compatible with the reference's
``src/liger_kernel/transformers/fused_linear_jsd.py:8-104``."""

from typing import Optional

import torch

from ..ops.fused_linear_jsd import LigerFusedLinearJSDFunction


class LigerFusedLinearJSD(torch.nn.Module):
    """Generalised Jensen-Shannon divergence between a student and a teacher language-model head, with both final
    projections fused in so that neither ``[BT, V]`` logits tensor is kept.

    ``jsd_beta`` in [0, 1] weights the teacher's distribution in the mixture (0: forward KL, 1: reverse KL);
    ``temperature`` divides both logits; tokens whose ``shift_labels`` entry equals ``ignore_index`` do not count.
    Shapes: student_input ``(BT, H)``, student_weight ``(V, H)``, teacher_input ``(BT, H')``, teacher_weight ``(V, H')``,
    shift_labels ``(BT,)`` or None; returns a scalar."""

    def __init__(self, jsd_beta=0.5, ignore_index=-100, temperature=1.0, accum_dtype: Optional[torch.dtype] = None):
        super().__init__()
        assert temperature != 0, "temperature cannot be 0."
        self.jsd_beta = jsd_beta
        self.temperature = temperature
        self.ignore_index = ignore_index
        self.accum_dtype = accum_dtype

    def forward(self, student_input: torch.Tensor, student_weight: torch.Tensor, teacher_input: torch.Tensor,
                teacher_weight: torch.Tensor, shift_labels: Optional[torch.LongTensor] = None):
        return LigerFusedLinearJSDFunction.apply(
            student_input, student_weight, teacher_input, teacher_weight, shift_labels, self.jsd_beta, self.ignore_index,
            self.temperature, self.accum_dtype,
        )
