"""GRPO and its relatives on the hidden states in front of the lm_head, without logits.

The reference (``src/liger_kernel/chunked_loss/fused_linear_ppo.py:161-586``, ``grpo_loss.py:100-536``) obtains the
log-probability of every sampled token with a vocabulary-chunked matmul of its own and evaluates the clipped-ratio loss under
``torch.compile``, chunk by chunk.  Here the per-token log-probabilities come from this library's tensor-core sweeps: the fused
head with ``reduction="none"`` when the sampling temperature is 1, the fused *scaled* cross-entropy (logits divided by the
temperature inside the sweep's epilogue) otherwise.  The loss is arithmetic on ``[B, T]`` tensors in torch; autograd hands the
per-token upstream gradients back to the operator's backward, which recomputes the logit tiles and projects them.

Loss types: ``grpo``, ``bnpo``, ``dr_grpo``, ``dapo``, ``cispo``, ``luspo``, ``sapo``, ``vespo``; token- or sequence-level
importance ratios; KL penalty to a reference policy (k3 estimator) with or without the importance-sampling correction; the
two-sided ``delta`` clamp; the vLLM importance-sampling ratio.  ``compiled`` and ``chunk_size`` are accepted and mean nothing
here.
"""

from __future__ import annotations

import torch

from ..ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction
from ..ops.fused_linear_scaled_cross_entropy import LigerFusedLinearScaledCrossEntropyFunction
from .preference import _ApplyMixin

_IGNORE = -100


def selected_token_logps(_input, weight, selected_token_ids, attention_mask, bias=None, temperature=1.0):
    """``log softmax(logits / temperature)[token]`` per position, ``[B, T]`` fp32; with an ``attention_mask`` the positions
    outside it are not evaluated (they read 0 and receive no gradient)."""
    b, t, h = _input.shape
    ids = selected_token_ids
    if attention_mask is not None:
        ids = torch.where(attention_mask.bool(), ids, torch.full_like(ids, _IGNORE))
    ids = ids.reshape(b * t)
    x = _input.reshape(b * t, h)
    if temperature == 1.0:
        nll = LigerFusedLinearCrossEntropyFunction.apply(x, weight, ids, bias, None, _IGNORE, 0.0, 0.0, "none")[0]
    else:
        if bias is not None:
            raise NotImplementedError("a head bias together with a sampling temperature other than 1 is not supported")
        nll = LigerFusedLinearScaledCrossEntropyFunction.apply(x, weight, ids, float(temperature), _IGNORE, 1, False)
    return -nll.float().view(b, t)


def _soft_gate(ratio, temperature):
    """SAPO's smooth replacement of the clip (``grpo_loss.py:56-76``)."""
    if temperature <= 0:
        raise ValueError("sapo_temperature must be > 0.")
    return torch.sigmoid(temperature * (ratio - 1)) * 4 / temperature


@torch.no_grad()
def _gamma_weights(advantages, log_ratio, mask, is_ratio, k_pos, lambda_pos, k_neg, lambda_neg):
    """VESPO's sequence-level weight phi(w) = e^lambda * w^k * e^(-lambda w) of the importance ratio w (phi(1) = 1), evaluated in
    log space and used as a constant (``grpo_loss.py:16-53``); shape ``[B, 1]``."""
    import math

    floor = math.log(1e-8)
    seq = (torch.clamp(log_ratio, -20.0, 20.0) * mask).sum(-1, keepdim=True)
    if is_ratio is not None:
        seq = seq + torch.clamp(torch.log(is_ratio), floor, 20.0).sum(-1, keepdim=True)
    log_w = torch.clamp(seq, floor, 20.0)
    w = torch.exp(log_w)
    nonneg = advantages.unsqueeze(-1) >= 0
    k = torch.where(nonneg, k_pos, k_neg)
    lam = torch.where(nonneg, lambda_pos, lambda_neg).clamp(min=1e-4)
    return torch.exp(lam + k * log_w - lam * w).nan_to_num(nan=0.0, posinf=0.0, neginf=0.0)


def _dapo_normalizer(attention_mask, num_items_in_batch):
    """Active tokens per process (``fused_linear_ppo.py:438-473``): given from outside, or counted over all ranks."""
    world = 1
    ranks = torch.distributed.is_available() and torch.distributed.is_initialized()
    if ranks:
        world = torch.distributed.get_world_size()
    if num_items_in_batch is not None:
        n = torch.as_tensor(num_items_in_batch, device=attention_mask.device).to(torch.float32)
    else:
        n = attention_mask.to(torch.float32).sum()
        if ranks:
            n = n.clone()
            torch.distributed.all_reduce(n)
    return torch.clamp(n / world, min=1.0)


def grpo_loss_fn(per_token_logps, attention_mask, advantages, ref_per_token_logps=None, old_per_token_logps=None,
                 epsilon_low=0.2, epsilon_high=0.2, beta=0.04, loss_type="dapo", max_completion_length=None,
                 importance_sampling_level="token", sapo_temperature_pos=1.0, sapo_temperature_neg=1.05, vllm_is_ratio=None,
                 delta=None, use_bias_correction_kl=False, num_items_in_batch=None, vespo=(2.0, 3.0, 3.0, 2.0)):
    """The clipped-ratio policy loss of GRPOTrainer on a whole batch (``grpo_loss.py:100-281``).  Returns
    ``(loss, [kl (if beta != 0), clip_ratio])``."""
    if importance_sampling_level not in ("token", "sequence"):
        raise ValueError(f"Unknown importance sampling level: {importance_sampling_level}. Possible values are 'token' and 'sequence'.")
    if importance_sampling_level == "sequence" and loss_type in ("cispo", "sapo", "vespo"):
        raise ValueError(f"Sequence-level importance sampling is not supported for loss_type='{loss_type}'. "
                         "Use importance_sampling_level='token' instead.")
    mask = attention_mask.to(per_token_logps.dtype)
    adv = advantages.to(per_token_logps.dtype).unsqueeze(1)
    if ref_per_token_logps is None:
        ref_per_token_logps = per_token_logps.detach()
    old = per_token_logps.detach() if old_per_token_logps is None else old_per_token_logps.float()
    log_ratio = per_token_logps - old
    if importance_sampling_level == "sequence":
        log_w = ((log_ratio * mask).sum(-1) / mask.sum(-1).clamp(min=1.0)).unsqueeze(-1)
    else:
        log_w = log_ratio
    ratio = torch.exp(log_w)
    lower = upper = torch.zeros_like(ratio, dtype=torch.bool)
    if loss_type == "cispo":
        clipped = torch.clamp(ratio, max=epsilon_high).detach()
        upper = ratio > epsilon_high
        per_token = -clipped * adv * per_token_logps
    elif loss_type == "vespo":
        phi = _gamma_weights(advantages.to(per_token_logps.dtype), log_ratio, mask, vllm_is_ratio, *vespo)
        per_token = -phi * adv * per_token_logps
    elif loss_type == "sapo":
        positive = adv.expand_as(ratio) > 0
        per_token = -torch.where(positive, _soft_gate(ratio, sapo_temperature_pos), _soft_gate(ratio, sapo_temperature_neg)) * adv
    else:
        lo, hi = 1 - epsilon_low, 1 + epsilon_high
        clipped = torch.clamp(ratio, lo, hi)
        lower, upper = ratio < lo, ratio > hi
        unclipped = ratio if delta is None else torch.clamp(ratio, max=delta)
        per_token = -torch.min(unclipped * adv, clipped * adv)
    if vllm_is_ratio is not None and loss_type != "vespo":      # vespo folds that correction into its sequence weight
        per_token = per_token * vllm_is_ratio
    kl = None
    if beta != 0.0:
        d = ref_per_token_logps.float() - per_token_logps
        kl = torch.exp(d) - d - 1.0                         # k3 estimate of KL(policy || reference)
        if use_bias_correction_kl:
            kl = kl * torch.exp(log_w)
        per_token = per_token + beta * kl
    rows = attention_mask.shape[0]
    if loss_type in ("grpo", "sapo"):
        loss = ((per_token * mask).sum(-1) / mask.sum(-1).clamp(min=1.0)).sum() / rows
    elif loss_type == "bnpo":
        loss = (per_token * mask).sum() / mask.sum().clamp(min=1.0)
    elif loss_type == "dr_grpo":
        if max_completion_length is None:
            raise ValueError("max_completion_length must be provided for loss_type 'dr_grpo'")
        loss = (per_token * mask).sum() / (rows * max_completion_length)
    elif loss_type in ("dapo", "cispo", "vespo"):
        loss = (per_token * mask).sum() / _dapo_normalizer(attention_mask, num_items_in_batch)
    elif loss_type == "luspo":
        weighted = per_token * mask.sum(1, keepdim=True)
        loss = weighted.sum() / (rows * weighted.shape[1])
    else:
        raise ValueError(f"Unknown loss type: {loss_type}")
    metrics = []
    total = mask.sum().clamp(min=1.0)
    if kl is not None:
        metrics.append(((kl * mask).sum() / total).detach())
    is_clipped = ((lower & (adv < 0)) | (upper & (adv > 0))).expand_as(mask)
    metrics.append(((is_clipped * mask).sum() / total).detach())
    return loss, metrics


class LigerFusedLinearGRPOFunction(_ApplyMixin):
    """Positional call surface of the reference's Function (``grpo_loss.py:283-416``); returns ``(loss, metrics)``."""

    @staticmethod
    def forward(_input, weight, selected_token_ids, attention_mask, advantages, bias=None, ref_per_token_logps=None,
                old_per_token_logps=None, ref_input=None, ref_weight=None, ref_bias=None, beta=0.04, epsilon_low=0.2,
                epsilon_high=0.2, loss_type="dapo", max_completion_length=None, importance_sampling_level="token",
                sapo_temperature_pos=1.0, sapo_temperature_neg=1.05, temperature=1.0, compiled=True, use_ref_model=True,
                chunk_size=1, vllm_is_ratio=None, delta=None, use_bias_correction_kl=False, vespo_k_pos=2.0, vespo_lambda_pos=3.0,
                vespo_k_neg=3.0, vespo_lambda_neg=2.0, num_items_in_batch=None):
        if _input.dim() != 3 or selected_token_ids.shape != _input.shape[:2] or attention_mask.shape != _input.shape[:2]:
            raise ValueError("expected _input [B, T, H], selected_token_ids [B, T] and attention_mask [B, T]")
        if use_ref_model:
            assert ref_per_token_logps is not None or ref_input is not None, (
                "If use_ref_model is True, ref_per_token_logps or ref_input must be provided")
        if loss_type == "dr_grpo":
            assert max_completion_length is not None, "max_completion_length must be provided for loss_type 'dr_grpo'"
        if vllm_is_ratio is not None:
            b, t = attention_mask.shape
            assert vllm_is_ratio.dim() in (1, 2), f"vllm_is_ratio must be 1D (B,) or 2D (B, T) / (B, 1), got {vllm_is_ratio.dim()}D"
            if vllm_is_ratio.dim() == 1:
                assert vllm_is_ratio.shape[0] == b, f"vllm_is_ratio shape must be ({b},), got {tuple(vllm_is_ratio.shape)}"
                vllm_is_ratio = vllm_is_ratio.unsqueeze(-1)
            else:
                assert vllm_is_ratio.shape[0] == b and vllm_is_ratio.shape[1] in (1, t), (
                    f"vllm_is_ratio shape must be ({b}, 1) or ({b}, {t}), got {tuple(vllm_is_ratio.shape)}")
        # "luspo" averages the per-token loss over every position, masked ones included (as the reference and TRL do), so
        # there every position has to be evaluated
        evaluated = None if loss_type == "luspo" else attention_mask
        logps = selected_token_logps(_input, weight, selected_token_ids, evaluated, bias, temperature)
        if use_ref_model and ref_per_token_logps is None:
            with torch.no_grad():
                ref_per_token_logps = selected_token_logps(ref_input, ref_weight, selected_token_ids, evaluated, ref_bias,
                                                           temperature)
        loss, metrics = grpo_loss_fn(
            logps, attention_mask, advantages, ref_per_token_logps if use_ref_model else None, old_per_token_logps, epsilon_low,
            epsilon_high, beta, loss_type, max_completion_length, importance_sampling_level, sapo_temperature_pos,
            sapo_temperature_neg, vllm_is_ratio, delta, use_bias_correction_kl, num_items_in_batch,
            (vespo_k_pos, vespo_lambda_pos, vespo_k_neg, vespo_lambda_neg))
        return loss, tuple(metrics)


class LigerFusedLinearGRPOLoss(torch.nn.Module):
    """``grpo_loss.py:418-536``: same constructor and ``forward`` arguments."""

    def __init__(self, beta=0.04, compiled=True, use_ref_model=True, chunk_size=1, epsilon_low=0.2, epsilon_high=0.2,
                 loss_type="dapo", max_completion_length=None, importance_sampling_level="token", sapo_temperature_pos=1.0,
                 sapo_temperature_neg=1.05, temperature=1.0, delta=None, use_bias_correction_kl=False, vespo_k_pos=2.0,
                 vespo_lambda_pos=3.0, vespo_k_neg=3.0, vespo_lambda_neg=2.0):
        super().__init__()
        if sapo_temperature_pos <= 0:
            raise ValueError(f"sapo_temperature_pos must be positive, got {sapo_temperature_pos}")
        if sapo_temperature_neg <= 0:
            raise ValueError(f"sapo_temperature_neg must be positive, got {sapo_temperature_neg}")
        if delta is not None and delta <= 0:
            raise ValueError(f"delta must be positive, got {delta}")
        self.beta, self.compiled, self.use_ref_model, self.chunk_size = beta, compiled, use_ref_model, chunk_size
        self.epsilon_low, self.epsilon_high, self.loss_type = epsilon_low, epsilon_high, loss_type
        self.max_completion_length, self.importance_sampling_level = max_completion_length, importance_sampling_level
        self.sapo_temperature_pos, self.sapo_temperature_neg, self.temperature = sapo_temperature_pos, sapo_temperature_neg, temperature
        self.delta, self.use_bias_correction_kl = delta, use_bias_correction_kl
        self.vespo = (vespo_k_pos, vespo_lambda_pos, vespo_k_neg, vespo_lambda_neg)

    def forward(self, _input, lin_weight, selected_token_ids, attention_mask, advantages, bias=None, ref_per_token_logps=None,
                old_per_token_logps=None, ref_input=None, ref_weight=None, ref_bias=None, vllm_is_ratio=None,
                num_items_in_batch=None):
        return LigerFusedLinearGRPOFunction.apply(
            _input, lin_weight, selected_token_ids, attention_mask, advantages, bias, ref_per_token_logps, old_per_token_logps,
            ref_input, ref_weight, ref_bias, self.beta, self.epsilon_low, self.epsilon_high, self.loss_type,
            self.max_completion_length, self.importance_sampling_level, self.sapo_temperature_pos, self.sapo_temperature_neg,
            self.temperature, self.compiled, self.use_ref_model, self.chunk_size, vllm_is_ratio, self.delta,
            self.use_bias_correction_kl, *self.vespo, num_items_in_batch)
