"""JSD distillation on the two heads' hidden states (``src/liger_kernel/chunked_loss/jsd_loss.py:9-200`` on the base of
``fused_linear_distillation.py:10-290``): ``weight_hard_loss * CE(student, labels) + weight_soft_loss * JSD_beta(student / T,
teacher / T)``, both normalised by the number of labels that are not ``ignore_index``.

The reference chunks the rows, materialises student and teacher logits per chunk and differentiates under ``torch.compile``.
Both terms exist in this library as fused operators with exactly these definitions: the hard term is the fused head with mean
reduction, the soft term the fused linear JSD (same mixture ``M = beta * teacher + (1 - beta) * student``, same limits at beta 0
and 1, same normaliser), so the distillation loss is their weighted sum.  ``compiled`` and ``chunk_size`` mean nothing here."""

from __future__ import annotations

import torch

from ..ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction
from ..ops.fused_linear_jsd import LigerFusedLinearJSDFunction as _HeadJSD
from .preference import _ApplyMixin


class LigerFusedLinearJSDFunction(_ApplyMixin):
    """Positional call surface of ``chunked_loss/jsd_loss.py:58-118``.  Inputs ``[BT, H]`` / ``[BT, H']``, weights ``[V, H]`` /
    ``[V, H']``, labels ``[BT]``."""

    @staticmethod
    def forward(student_input, student_weight, teacher_input, teacher_weight, true_labels, student_bias=None, teacher_bias=None,
                weight_hard_loss=0.5, weight_soft_loss=0.5, beta=0.5, ignore_index=-100, temperature=1.0, compiled=True,
                chunk_size=1024, return_soft_hard_loss=False):
        if student_bias is not None or teacher_bias is not None:
            raise NotImplementedError("head biases are not supported by the fused JSD distillation loss")
        if student_weight.shape[0] != teacher_weight.shape[0]:
            raise NotImplementedError("student and teacher must share a vocabulary size")
        # both terms are always evaluated and reported (the reference does the same); a term with weight zero is evaluated
        # without recording, i.e. as a forward-only call
        with torch.set_grad_enabled(torch.is_grad_enabled() and weight_hard_loss != 0):
            hard = LigerFusedLinearCrossEntropyFunction.apply(student_input, student_weight, true_labels, None, None, ignore_index,
                                                              0.0, 0.0, "mean")[0].float()
        with torch.set_grad_enabled(torch.is_grad_enabled() and weight_soft_loss != 0):
            soft = _HeadJSD.apply(student_input, student_weight, teacher_input, teacher_weight, true_labels, beta, ignore_index,
                                  temperature, None).float()
        loss = weight_hard_loss * hard + weight_soft_loss * soft
        if return_soft_hard_loss:
            return loss, soft.detach(), hard.detach()
        return loss


class LigerFusedLinearJSDLoss(torch.nn.Module):
    """``chunked_loss/jsd_loss.py:136-200``: same constructor and ``forward`` arguments."""

    def __init__(self, weight_hard_loss=0.5, weight_soft_loss=0.5, beta=0.5, ignore_index=-100, temperature=1.0, compiled=True,
                 chunk_size=1024, return_soft_hard_loss=False):
        super().__init__()
        assert temperature != 0, "Temperature cannot be 0."
        self.weight_hard_loss, self.weight_soft_loss, self.beta = weight_hard_loss, weight_soft_loss, beta
        self.ignore_index, self.temperature, self.compiled = ignore_index, temperature, compiled
        self.chunk_size, self.return_soft_hard_loss = chunk_size, return_soft_hard_loss

    def forward(self, student_input, student_weight, teacher_input, teacher_weight, true_labels, student_bias=None,
                teacher_bias=None):
        return LigerFusedLinearJSDFunction.apply(student_input, student_weight, teacher_input, teacher_weight, true_labels,
                                                 student_bias, teacher_bias, self.weight_hard_loss, self.weight_soft_loss, self.beta,
                                                 self.ignore_index, self.temperature, self.compiled, self.chunk_size,
                                                 self.return_soft_hard_loss)
