"""Preference losses on the hidden states in front of the lm_head, without logits.

The reference's ``chunked_loss`` losses (``src/liger_kernel/chunked_loss/fused_linear_preference.py:9-433``) walk over the batch
in chunks, materialise ``[chunk, T, V]`` logits with a matmul, take ``log_softmax`` and differentiate the chunk with
``torch.func.grad_and_value`` under ``torch.compile``.  All any of them needs from the ``V``-wide rows is the log-probability of
each target token, ``log p_t = x_t - lse_t``, and that is the per-row output of this library's fused head with
``reduction="none"`` (negated): the tensor-core sweep produces it in its epilogue and no logit ever reaches memory.  The pairwise
loss itself is arithmetic on ``[batch]`` vectors, done in torch; autograd hands the per-token upstream gradient back to the fused
head, whose backward recomputes the logit tiles and projects them (``reduction="none"`` with non-uniform per-token gradients is
part of that operator's contract, ``test/transformers/test_fused_linear_cross_entropy.py:1041-1094`` of the reference).

Inputs follow the reference: ``_input [B, T, H]`` with the chosen sequences in the first half of the batch and the rejected ones
in the second, ``target [B, T]``.  Results follow it too: ``(loss, (chosen_logps, rejected_logps, chosen_logits_mean,
rejected_logits_mean, nll_loss, *aux))``.  ``compiled`` and ``chunk_size`` are accepted and have no meaning here.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from ..ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction


def per_token_logps(_input, weight, target, bias=None, ignore_index=-100):
    """``log p(target_t)`` per position, ``[B, T]`` fp32, zero where ``target == ignore_index``; differentiable with respect to
    ``_input``, ``weight`` and ``bias`` through the fused head."""
    b, t, h = _input.shape
    rows = LigerFusedLinearCrossEntropyFunction.apply(_input.reshape(b * t, h), weight, target.reshape(b * t), bias, None,
                                                      ignore_index, 0.0, 0.0, "none")[0]
    return -rows.float().view(b, t)


def _logits_mean(_input, weight, bias, n_rows_total):
    """Mean of all logits of a block of sequences: sum_{r,v} x_r . w_v = (sum_r x_r) . (sum_v w_v), so two column sums and one dot
    product stand in for the reference's ``logits.sum()`` (``fused_linear_preference.py:389-392``)."""
    x_sum = _input.detach().float().sum(dim=(0, 1))
    total = torch.dot(x_sum, weight.detach().float().sum(dim=0))
    if bias is not None:
        total = total + bias.detach().float().sum() * (_input.shape[0] * _input.shape[1])
    return total / (n_rows_total * weight.shape[0])


def preference_forward(loss_fn, _input, weight, target, bias=None, ignore_index=-100, alpha=1.0, beta=0.1, compute_nll_loss=True,
                       nll_target=None, use_ref_model=False, ref_input=None, ref_weight=None, ref_bias=None,
                       average_log_prob=True, **loss_kwargs):
    """The common part (``LigerFusedLinearPreferenceBase.forward`` / ``_compute_loss``, ``:17-433``) on the whole batch at once."""
    if _input.dim() != 3 or target.dim() != 2 or _input.shape[:2] != target.shape:
        raise ValueError(f"expected _input [B, T, H] and target [B, T], got {tuple(_input.shape)} and {tuple(target.shape)}")
    if _input.shape[0] % 2 != 0:
        raise ValueError("the batch holds the chosen sequences followed by as many rejected ones: its size must be even")
    pairs = _input.shape[0] // 2
    mask = target != ignore_index
    logps = per_token_logps(_input, weight, target, bias, ignore_index)
    seq = logps.sum(-1)
    if average_log_prob:
        seq = seq / mask.sum(-1)
    chosen_logps, rejected_logps = seq[:pairs], seq[pairs:]

    nll = torch.zeros((), device=_input.device, dtype=torch.float32)
    if compute_nll_loss:
        if nll_target is None:
            nll = -logps[:pairs].sum() / mask[:pairs].sum()
        else:
            chosen_nll_target = nll_target[:pairs]
            h = _input.shape[-1]
            total = LigerFusedLinearCrossEntropyFunction.apply(_input[:pairs].reshape(-1, h), weight, chosen_nll_target.reshape(-1),
                                                               bias, None, ignore_index, 0.0, 0.0, "sum")[0]
            nll = total.float() / (chosen_nll_target != ignore_index).sum()

    if use_ref_model:
        with torch.no_grad():
            ref = per_token_logps(ref_input, ref_weight, target, ref_bias, ignore_index).sum(-1)
            if average_log_prob:
                ref = ref / mask.sum(-1)
        loss_kwargs["ref_chosen_logps"], loss_kwargs["ref_rejected_logps"] = ref[:pairs], ref[pairs:]

    outputs = loss_fn(chosen_logps, rejected_logps, pairs, beta=beta, **loss_kwargs)
    preference_loss, aux = (outputs[0], list(outputs[1:])) if isinstance(outputs, tuple) else (outputs, [])
    loss = alpha * nll + preference_loss
    with torch.no_grad():
        chosen_mean = _logits_mean(_input[:pairs], weight, bias, pairs * _input.shape[1])
        rejected_mean = _logits_mean(_input[pairs:], weight, bias, pairs * _input.shape[1])
    return loss, (chosen_logps.detach(), rejected_logps.detach(), chosen_mean, rejected_mean, nll.detach(),
                  *[a.detach() for a in aux])


# ---------------------------------------------------------------- the pairwise losses (arithmetic on [pairs] vectors)
def dpo_loss_fn(chosen_logps, rejected_logps, pairs, ref_chosen_logps=None, ref_rejected_logps=None, beta=0.1,
                loss_type="sigmoid", label_smoothing=0.0, discopop_tau=0.05):
    """Direct preference optimisation and its variants (``chunked_loss/dpo_loss.py:9-155``)."""
    zero = torch.zeros((), device=chosen_logps.device)
    c = chosen_logps - (zero if ref_chosen_logps is None else ref_chosen_logps)
    r = rejected_logps - (zero if ref_rejected_logps is None else ref_rejected_logps)
    chosen_rewards, rejected_rewards = beta * c, beta * r
    d = beta * (c - r)
    if loss_type == "sigmoid":
        per_pair = -F.logsigmoid(d)
    elif loss_type == "hinge":
        per_pair = torch.relu(1 - d)
    elif loss_type == "exo_pair":
        if label_smoothing <= 0.0:
            raise ValueError("label_smoothing must be > 0 for loss_type='exo_pair'. The EXO paper recommends 1e-3.")
        eps = torch.tensor(label_smoothing, device=d.device)
        per_pair = (torch.sigmoid(d) * (F.logsigmoid(d) - torch.log1p(-eps))
                    + torch.sigmoid(-d) * (F.logsigmoid(-d) - torch.log(eps)))
    elif loss_type == "nca_pair":
        per_pair = -F.logsigmoid(chosen_rewards) - 0.5 * F.logsigmoid(-chosen_rewards) - 0.5 * F.logsigmoid(-rejected_rewards)
    elif loss_type == "robust":
        if not (0.0 <= label_smoothing < 0.5):
            raise ValueError(f"label_smoothing must lie in [0.0, 0.5) for loss_type='robust'. Got {label_smoothing}.")
        per_pair = (-(1 - label_smoothing) * F.logsigmoid(d) + label_smoothing * F.logsigmoid(-d)) / (1 - 2 * label_smoothing)
    elif loss_type == "bco_pair":
        per_pair = -F.logsigmoid(chosen_rewards) - F.logsigmoid(-rejected_rewards)
    elif loss_type == "sppo_hard":
        per_pair = (c - 0.5 / beta) ** 2 + (r + 0.5 / beta) ** 2
    elif loss_type == "apo_zero":
        per_pair = (1 - torch.sigmoid(beta * c)) + torch.sigmoid(beta * r)
    elif loss_type == "apo_down":
        per_pair = torch.sigmoid(beta * c) + (1 - torch.sigmoid(beta * (c - r)))
    elif loss_type == "discopop":
        m = torch.sigmoid(d / discopop_tau)
        per_pair = -F.logsigmoid(d) * (1 - m) + torch.exp(-d) * m
    elif loss_type == "ipo":
        raise NotImplementedError("loss_type='ipo' needs per-sample completion-token counts; the reference does not support it either")
    else:
        raise ValueError(f"Unsupported loss_type: {loss_type}. Supported types are: sigmoid, hinge, exo_pair, nca_pair, "
                         "robust, bco_pair, sppo_hard, apo_zero, apo_down, discopop")
    return per_pair.sum() / pairs, chosen_rewards, rejected_rewards


def orpo_loss_fn(chosen_logps, rejected_logps, pairs, beta=0.1):
    """Odds-ratio preference optimisation (``chunked_loss/orpo_loss.py:8-43``); the log-probabilities are per-token averages."""
    log_odds = (chosen_logps - rejected_logps) - (torch.log1p(-torch.exp(chosen_logps)) - torch.log1p(-torch.exp(rejected_logps)))
    ratio = F.logsigmoid(log_odds)
    return (-beta * ratio.sum() / pairs, beta * chosen_logps, beta * rejected_logps, ratio.sum() / pairs, log_odds.sum() / pairs)


def simpo_loss_fn(chosen_logps, rejected_logps, pairs, beta=0.1, gamma=0.5, label_smoothing=0.0):
    """SimPO (``chunked_loss/simpo_loss.py:8-48``): reference-free, length-normalised, with a target margin gamma."""
    z = beta * (chosen_logps - rejected_logps) - gamma
    loss = (-F.logsigmoid(z) * (1 - label_smoothing) - F.logsigmoid(-z) * label_smoothing).sum() / pairs
    return loss, beta * chosen_logps, beta * rejected_logps


def cpo_loss_fn(chosen_logps, rejected_logps, pairs, beta=0.1, label_smoothing=0.0):
    """Contrastive preference optimisation (``chunked_loss/cpo_loss.py:8-40``)."""
    z = beta * (chosen_logps - rejected_logps)
    loss = (-F.logsigmoid(z) * (1 - label_smoothing) - F.logsigmoid(-z) * label_smoothing).sum() / pairs
    return loss, beta * chosen_logps, beta * rejected_logps


def kto_loss_fn(log_probs, preference_labels, batch, ref_log_probs=None, beta=0.1, kl=None):
    """Kahneman-Tversky optimisation on unpaired samples (``chunked_loss/kto_loss.py:8-70``): a desirable sample is pushed above
    the KL reference point, an undesirable one below it."""
    ratios = log_probs if ref_log_probs is None else log_probs - ref_log_probs
    sign = torch.where(preference_labels, 1.0, -1.0)
    z = ratios if kl is None else ratios - kl
    loss = (1 - torch.sigmoid(beta * z * sign)).sum() / batch
    rewards = beta * ratios
    return loss, (rewards * preference_labels).sum(), (rewards * ~preference_labels).sum()


def unpaired_preference_forward(loss_fn, _input, weight, target, preference_labels, bias=None, ignore_index=-100, beta=0.1,
                                use_ref_model=False, ref_input=None, ref_weight=None, ref_bias=None, average_log_prob=False,
                                **loss_kwargs):
    """``LigerFusedLinearUnpairedPreferenceBase`` (``chunked_loss/fused_linear_unpaired_preference.py:9-341``) on the whole batch at
    once: every sequence carries its own desirable / undesirable label.  The per-class sums are sums over the samples of that
    class (what the reference's chunk loop accumulates with its default chunk size of one sample)."""
    if _input.dim() != 3 or target.dim() != 2 or _input.shape[:2] != target.shape:
        raise ValueError(f"expected _input [B, T, H] and target [B, T], got {tuple(_input.shape)} and {tuple(target.shape)}")
    if preference_labels is None or preference_labels.shape != (_input.shape[0],):
        raise ValueError("preference_labels must hold one boolean per sequence")
    labels = preference_labels.to(device=_input.device, dtype=torch.bool)
    mask = target != ignore_index
    seq = per_token_logps(_input, weight, target, bias, ignore_index).sum(-1)
    if average_log_prob:
        seq = seq / mask.sum(-1)
    if use_ref_model:
        with torch.no_grad():
            ref = per_token_logps(ref_input, ref_weight, target, ref_bias, ignore_index).sum(-1)
            if average_log_prob:
                ref = ref / mask.sum(-1)
        loss_kwargs["ref_log_probs"] = ref
    outputs = loss_fn(seq, labels, _input.shape[0], beta=beta, **loss_kwargs)
    loss, aux = (outputs[0], list(outputs[1:])) if isinstance(outputs, tuple) else (outputs, [])
    with torch.no_grad():
        w_sum = weight.detach().float().sum(dim=0)
        row_sums = _input.detach().float().sum(dim=1) @ w_sum                        # [B]: sum of all logits of a sequence
        if bias is not None:
            row_sums = row_sums + bias.detach().float().sum() * _input.shape[1]
        chosen_logits_sum, rejected_logits_sum = (row_sums * labels).sum(), (row_sums * ~labels).sum()
        chosen_logps_sum, rejected_logps_sum = (seq.detach() * labels).sum(), (seq.detach() * ~labels).sum()
    return loss, (chosen_logps_sum, rejected_logps_sum, chosen_logits_sum, rejected_logits_sum, *[a.detach() for a in aux])


# ---------------------------------------------------------------- call surface of the reference's classes
class _ApplyMixin:
    """The reference exposes autograd Functions and calls them positionally through ``.apply``
    (``chunked_loss/functional.py:10-17``); these classes keep that spelling.  Gradients flow through the fused head's own
    autograd Function, so nothing here needs to be one."""

    @classmethod
    def apply(cls, *args, **kwargs):
        return cls.forward(*args, **kwargs)


class LigerFusedLinearDPOFunction(_ApplyMixin):
    @staticmethod
    def forward(_input, weight, target, bias=None, ref_input=None, ref_weight=None, ref_bias=None, ignore_index=-100, beta=0.1,
                compute_nll_loss=False, compiled=True, use_ref_model=True, average_log_prob=False, chunk_size=1,
                loss_type="sigmoid", label_smoothing=0.0, discopop_tau=0.05, alpha=1.0):
        return preference_forward(dpo_loss_fn, _input, weight, target, bias, ignore_index, alpha, beta, compute_nll_loss, None,
                                  use_ref_model, ref_input, ref_weight, ref_bias, average_log_prob, loss_type=loss_type,
                                  label_smoothing=label_smoothing, discopop_tau=discopop_tau)


class LigerFusedLinearORPOFunction(_ApplyMixin):
    @staticmethod
    def forward(_input, weight, target, bias=None, ignore_index=-100, beta=0.1, compute_nll_loss=True, nll_target=None,
                compiled=True, chunk_size=1):
        return preference_forward(orpo_loss_fn, _input, weight, target, bias, ignore_index, 1.0, beta, compute_nll_loss,
                                  nll_target, average_log_prob=True)


class LigerFusedLinearSimPOFunction(_ApplyMixin):
    @staticmethod
    def forward(_input, weight, target, bias=None, ignore_index=-100, beta=0.1, alpha=1.0, label_smoothing=0.0,
                compute_nll_loss=False, compiled=True, gamma=0.5, chunk_size=1):
        return preference_forward(simpo_loss_fn, _input, weight, target, bias, ignore_index, alpha, beta, compute_nll_loss,
                                  average_log_prob=True, gamma=gamma, label_smoothing=label_smoothing)


class LigerFusedLinearCPOFunction(_ApplyMixin):
    @staticmethod
    def forward(_input, weight, target, bias=None, ignore_index=-100, beta=0.1, alpha=1.0, label_smoothing=0.0,
                compute_nll_loss=True, compiled=True, average_log_prob=False, chunk_size=1):
        return preference_forward(cpo_loss_fn, _input, weight, target, bias, ignore_index, alpha, beta, compute_nll_loss,
                                  average_log_prob=average_log_prob, label_smoothing=label_smoothing)


class LigerFusedLinearKTOFunction(_ApplyMixin):
    @staticmethod
    def forward(_input, weight, target, preference_labels, bias=None, ref_input=None, ref_weight=None, ref_bias=None, kl=None,
                ignore_index=-100, beta=0.1, compiled=True, use_ref_model=True, average_log_prob=False, chunk_size=1):
        return unpaired_preference_forward(kto_loss_fn, _input, weight, target, preference_labels, bias, ignore_index, beta,
                                           use_ref_model, ref_input, ref_weight, ref_bias, average_log_prob, kl=kl)


class LigerFusedLinearKTOLoss(torch.nn.Module):
    """``chunked_loss/kto_loss.py:140-210``: note the argument order of ``forward`` (``_input`` before ``lin_weight``)."""

    def __init__(self, ignore_index=-100, beta=0.1, compiled=True, use_ref_model=False, average_log_prob=False, chunk_size=1):
        super().__init__()
        self.ignore_index, self.beta, self.compiled = ignore_index, beta, compiled
        self.use_ref_model, self.average_log_prob, self.chunk_size = use_ref_model, average_log_prob, chunk_size

    def forward(self, _input, lin_weight, target, bias=None, preference_labels=None, ref_input=None, ref_weight=None,
                ref_bias=None, kl=None):
        return LigerFusedLinearKTOFunction.apply(_input, lin_weight, target, preference_labels, bias, ref_input, ref_weight,
                                                 ref_bias, kl, self.ignore_index, self.beta, self.compiled, self.use_ref_model,
                                                 self.average_log_prob, self.chunk_size)


class LigerFusedLinearDPOLoss(torch.nn.Module):
    """``chunked_loss/dpo_loss.py:233-331``: same constructor, same ``forward(lin_weight, _input, target, bias, ref_input,
    ref_weight, ref_bias)``."""

    _SUPPORTED_LOSS_TYPES = {"sigmoid", "hinge", "exo_pair", "nca_pair", "robust", "bco_pair", "sppo_hard", "apo_zero",
                             "apo_down", "discopop"}

    def __init__(self, ignore_index=-100, beta=0.1, alpha=1.0, compute_nll_loss=False, compiled=True, use_ref_model=True,
                 average_log_prob=False, chunk_size=1, loss_type="sigmoid", label_smoothing=0.0, discopop_tau=0.05):
        super().__init__()
        if loss_type not in self._SUPPORTED_LOSS_TYPES:
            raise ValueError(f"Unsupported loss_type: {loss_type}. Supported types are: {self._SUPPORTED_LOSS_TYPES}")
        if loss_type == "exo_pair" and label_smoothing <= 0.0:
            raise ValueError("label_smoothing must be > 0 for loss_type='exo_pair'. The EXO paper recommends 1e-3.")
        if loss_type == "robust" and not (0.0 <= label_smoothing < 0.5):
            raise ValueError(f"label_smoothing must lie in [0.0, 0.5) for loss_type='robust'. Got {label_smoothing}.")
        self.ignore_index, self.beta, self.alpha = ignore_index, beta, alpha
        self.compute_nll_loss, self.compiled, self.use_ref_model = compute_nll_loss, compiled, use_ref_model
        self.average_log_prob, self.chunk_size, self.loss_type = average_log_prob, chunk_size, loss_type
        self.label_smoothing, self.discopop_tau = label_smoothing, discopop_tau

    def forward(self, lin_weight, _input, target, bias=None, ref_input=None, ref_weight=None, ref_bias=None):
        return LigerFusedLinearDPOFunction.apply(_input, lin_weight, target, bias, ref_input, ref_weight, ref_bias,
                                                 self.ignore_index, self.beta, self.compute_nll_loss, self.compiled,
                                                 self.use_ref_model, self.average_log_prob, self.chunk_size, self.loss_type,
                                                 self.label_smoothing, self.discopop_tau, self.alpha)


class LigerFusedLinearORPOLoss(torch.nn.Module):
    """``chunked_loss/orpo_loss.py:97-144``."""

    def __init__(self, ignore_index=-100, beta=0.1, compute_nll_loss=True, compiled=True, chunk_size=1):
        super().__init__()
        self.ignore_index, self.beta, self.compute_nll_loss = ignore_index, beta, compute_nll_loss
        self.compiled, self.chunk_size = compiled, chunk_size

    def forward(self, lin_weight, _input, target, bias=None, nll_target=None):
        return LigerFusedLinearORPOFunction.apply(_input, lin_weight, target, bias, self.ignore_index, self.beta,
                                                  self.compute_nll_loss, nll_target, self.compiled, self.chunk_size)


class LigerFusedLinearSimPOLoss(torch.nn.Module):
    """``chunked_loss/simpo_loss.py:108-165``."""

    def __init__(self, ignore_index=-100, beta=0.1, alpha=1.0, label_smoothing=0.0, compute_nll_loss=True, compiled=True,
                 gamma=0.5, chunk_size=1):
        super().__init__()
        self.ignore_index, self.beta, self.alpha, self.label_smoothing = ignore_index, beta, alpha, label_smoothing
        self.compute_nll_loss, self.compiled, self.gamma, self.chunk_size = compute_nll_loss, compiled, gamma, chunk_size

    def forward(self, lin_weight, _input, target, bias=None):
        return LigerFusedLinearSimPOFunction.apply(_input, lin_weight, target, bias, self.ignore_index, self.beta, self.alpha,
                                                   self.label_smoothing, self.compute_nll_loss, self.compiled, self.gamma,
                                                   self.chunk_size)


class LigerFusedLinearCPOLoss(torch.nn.Module):
    """``chunked_loss/cpo_loss.py:100-157``."""

    def __init__(self, ignore_index=-100, beta=0.1, alpha=1.0, label_smoothing=0.0, compute_nll_loss=True, compiled=True,
                 average_log_prob=False, chunk_size=1):
        super().__init__()
        self.ignore_index, self.beta, self.alpha, self.label_smoothing = ignore_index, beta, alpha, label_smoothing
        self.compute_nll_loss, self.compiled, self.average_log_prob = compute_nll_loss, compiled, average_log_prob
        self.chunk_size = chunk_size

    def forward(self, lin_weight, _input, target, bias=None):
        return LigerFusedLinearCPOFunction.apply(_input, lin_weight, target, bias, self.ignore_index, self.beta, self.alpha,
                                                 self.label_smoothing, self.compute_nll_loss, self.compiled,
                                                 self.average_log_prob, self.chunk_size)
