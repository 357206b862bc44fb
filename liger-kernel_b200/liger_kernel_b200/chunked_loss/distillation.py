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


# ---------------------------------------------------------------- cosine-similarity distillation, without logits
class _Gram(torch.autograd.Function):
    """``A^T B`` for two tall matrices that share their row count (the vocabulary), accumulated in fp32 over row blocks so that no
    fp32 copy of a whole weight matrix is ever made; backward is two more such products."""

    BLOCK = 16384

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        g = torch.zeros(a.shape[1], b.shape[1], dtype=torch.float32, device=a.device)
        for r in range(0, a.shape[0], _Gram.BLOCK):
            g.addmm_(a[r:r + _Gram.BLOCK].float().t(), b[r:r + _Gram.BLOCK].float())
        return g

    @staticmethod
    def backward(ctx, dg):
        a, b = ctx.saved_tensors
        da = db = None
        if ctx.needs_input_grad[0]:
            da = torch.empty_like(a)
            for r in range(0, a.shape[0], _Gram.BLOCK):
                da[r:r + _Gram.BLOCK] = (b[r:r + _Gram.BLOCK].float() @ dg.t()).to(a.dtype)
        if ctx.needs_input_grad[1]:
            db = torch.empty_like(b)
            for r in range(0, b.shape[0], _Gram.BLOCK):
                db[r:r + _Gram.BLOCK] = (a[r:r + _Gram.BLOCK].float() @ dg).to(b.dtype)
        return da, db


def cosine_rows(student_input, student_weight, teacher_input, teacher_weight):
    """Cosine similarity between the student's and the teacher's logit rows, ``[BT]`` fp32, without forming a logit:
    ``sum_v s_v t_v = x_s (W_s^T W_t) x_t^T`` and likewise for the two squared norms, so three ``H x H'`` Gram matrices (plain
    GEMMs over the vocabulary) and three row-wise quadratic forms replace the two ``[BT, V]`` logit matrices.  The cost is
    O(V H H') + O(BT H H') instead of O(BT V (H + H')).  The temperature of the reference's signature cancels in a cosine."""
    with torch.no_grad():
        g_tt = _Gram.apply(teacher_weight, teacher_weight)
        xt = teacher_input.float()
        tt = ((xt @ g_tt) * xt).sum(-1)
    g_ss = _Gram.apply(student_weight, student_weight)
    g_st = _Gram.apply(student_weight, teacher_weight.detach())
    xs = student_input.float()
    ss = ((xs @ g_ss) * xs).sum(-1)
    st = ((xs @ g_st) * xt).sum(-1)
    eps = 1e-12                                    # F.normalize's floor on each norm
    return st / (ss.clamp_min(0).sqrt().clamp_min(eps) * tt.clamp_min(0).sqrt().clamp_min(eps))


class LigerFusedLinearCosineSimilarityFunction(_ApplyMixin):
    """Positional call surface of ``chunked_loss/cosine_similarity_loss.py:10-89``: ``weight_hard_loss * CE + weight_soft_loss *
    beta * sum_rows (1 - cos) / n_valid`` (the soft term runs over every row, as in the reference, and is divided by the number
    of labels that are not ``ignore_index``)."""

    @staticmethod
    def forward(student_input, student_weight, teacher_input, teacher_weight, true_labels, student_bias=None, teacher_bias=None,
                weight_hard_loss=0.5, weight_soft_loss=0.5, beta=0.5, ignore_index=-100, temperature=1.0, compiled=True,
                chunk_size=1024, return_soft_hard_loss=False):
        if student_bias is not None or teacher_bias is not None:
            raise NotImplementedError("head biases are not supported by the fused cosine-similarity distillation loss")
        if student_weight.shape[0] != teacher_weight.shape[0]:
            raise NotImplementedError("student and teacher must share a vocabulary size")
        with torch.set_grad_enabled(torch.is_grad_enabled() and weight_hard_loss != 0):
            hard = LigerFusedLinearCrossEntropyFunction.apply(student_input, student_weight, true_labels, None, None, ignore_index,
                                                              0.0, 0.0, "mean")[0].float()
        n_valid = (true_labels != ignore_index).sum().clamp_min(1)
        with torch.set_grad_enabled(torch.is_grad_enabled() and weight_soft_loss != 0):
            cos = cosine_rows(student_input, student_weight, teacher_input, teacher_weight)
            soft = beta * (1 - cos).sum() / n_valid
        loss = weight_hard_loss * hard + weight_soft_loss * soft
        if return_soft_hard_loss:
            return loss, soft.detach(), hard.detach()
        return loss


class LigerFusedLinearCosineSimilarityLoss(torch.nn.Module):
    """``chunked_loss/cosine_similarity_loss.py:92-143``: same constructor and ``forward`` arguments."""

    def __init__(self, weight_hard_loss=0.5, weight_soft_loss=0.5, beta=0.5, ignore_index=-100, temperature=1.0, compiled=True,
                 chunk_size=1024, return_soft_hard_loss=False):
        super().__init__()
        assert temperature != 0, "Temperature cannot be 0."
        self.weight_hard_loss, self.weight_soft_loss, self.beta = weight_hard_loss, weight_soft_loss, beta
        self.ignore_index, self.temperature, self.compiled = ignore_index, temperature, compiled
        self.chunk_size, self.return_soft_hard_loss = chunk_size, return_soft_hard_loss

    def forward(self, student_input, student_weight, teacher_input, teacher_weight, true_labels, student_bias=None,
                teacher_bias=None):
        return LigerFusedLinearCosineSimilarityFunction.apply(
            student_input, student_weight, teacher_input, teacher_weight, true_labels, student_bias, teacher_bias,
            self.weight_hard_loss, self.weight_soft_loss, self.beta, self.ignore_index, self.temperature, self.compiled,
            self.chunk_size, self.return_soft_hard_loss)
