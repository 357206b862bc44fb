"""CPU oracles for the two sibling losses of the fused linear cross-entropy path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product path may import this file; it exists so that tests (and the
generator of the golden vectors) can check results against closed-form fp64 math.

* ``fused_linear_jsd_oracle``: generalised Jensen-Shannon divergence between a student head and a teacher head
  (reference: ``src/liger_kernel/ops/fused_linear_jsd.py:23-157`` for the chunk loop and the chain rule through
  ``log_softmax``, ``src/liger_kernel/ops/jsd.py:12-93`` for the per-element terms).
* ``fused_linear_scaled_ce_oracle``: per-token negative log-likelihood and entropy at a temperature
  (reference: ``src/liger_kernel/ops/fused_linear_scaled_cross_entropy.py:50-93``).

Pinned to outputs of the reference itself (``tests/golden/jsd_*.npz``, ``tests/golden/sce_*.npz``, produced by
``tests/golden/make_golden.py``); ``tests/test_oracle.py`` holds the comparison.
"""

from typing import NamedTuple, Optional

import torch


def _round(t, dtype):
    return t if dtype is None else t.to(dtype).to(t.dtype)


class JSDResult(NamedTuple):
    loss: torch.Tensor                 # scalar
    loss_rows: torch.Tensor            # [BT] per-token contribution (already divided by the token count)
    grad_input: torch.Tensor           # [BT, H] with respect to the student's hidden states
    grad_weight: torch.Tensor          # [V, H] with respect to the student's head
    grad_logits: torch.Tensor          # [BT, V] with respect to the student's (unscaled) logits


def fused_linear_jsd_oracle(student_input, student_weight, teacher_input, teacher_weight, shift_labels=None, jsd_beta=0.5,
                            ignore_index=-100, temperature=1.0, grad_output=1.0, round_logits_to: Optional[torch.dtype] = None,
                            round_dlogits_to: Optional[torch.dtype] = None, compute_dtype=torch.float64) -> JSDResult:
    """With X = log_softmax(student logits / T) (log Q) and Y = log_softmax(teacher logits / T) (log P), per element
    (``ops/jsd.py:54-90``):

      beta = 0 (forward KL):  loss = P (Y - X),                         dX = -P
      beta = 1 (reverse KL):  loss = Q (X - Y),                         dX = loss + Q
      otherwise, M = beta P + (1 - beta) Q:
                              loss = beta P Y + (1 - beta) Q X - M log M,   dX = (1 - beta) Q (X - log M)

    all divided by the number of tokens whose label is not ``ignore_index`` (every token when no labels are given);
    rows with an ignored label contribute nothing.  The chain through ``log_softmax`` and the temperature
    (``ops/fused_linear_jsd.py:118-122``): d logits = (dX - Q * sum_k dX_k) / T.  ``round_logits_to`` rounds both
    matrix products to a 16-bit type first, ``round_dlogits_to`` rounds the logit gradient before the two projections,
    as the reference and the product do for 16-bit inputs."""
    xs, ws = student_input.to(compute_dtype), student_weight.to(compute_dtype)
    xt, wt = teacher_input.to(compute_dtype), teacher_weight.to(compute_dtype)
    n_rows = xs.shape[0]
    zs = _round(xs @ ws.T, round_logits_to) / temperature
    zt = _round(xt @ wt.T, round_logits_to) / temperature
    X, Y = torch.log_softmax(zs, dim=-1), torch.log_softmax(zt, dim=-1)
    Q, P = X.exp(), Y.exp()
    if shift_labels is not None:
        live = (shift_labels != ignore_index)
        n = int(live.sum())
    else:
        live = torch.ones(n_rows, dtype=torch.bool)
        n = n_rows
    beta = float(jsd_beta)
    if beta == 0.0:
        loss = P * (Y - X)
        dX = -P
    elif beta == 1.0:
        loss = Q * (X - Y)
        dX = loss + Q
    else:
        M = beta * P + (1 - beta) * Q
        log_m = M.log()
        loss = beta * P * Y + (1 - beta) * Q * X - M * log_m
        dX = (1 - beta) * Q * (X - log_m)
    mask = live.to(compute_dtype)[:, None]
    scale = 1.0 / n if n > 0 else 0.0
    loss = torch.nan_to_num(loss) * mask * scale          # 0 * log 0 terms of fully underflowed classes
    dX = torch.nan_to_num(dX) * mask * scale
    dz = (dX - Q * dX.sum(dim=-1, keepdim=True)) / temperature
    dz = _round(dz, round_dlogits_to)
    go = float(grad_output)
    return JSDResult(loss=loss.sum(), loss_rows=loss.sum(dim=-1), grad_input=(dz @ ws) * go, grad_weight=(dz.T @ xs) * go,
                     grad_logits=dz * go)


class ScaledCEResult(NamedTuple):
    nll: torch.Tensor                  # [M] -log softmax(z / T)[target], 0 on ignored tokens
    entropy: torch.Tensor              # [M] entropy of softmax(z / T), 0 on ignored tokens
    grad_input: torch.Tensor           # [M, H]
    grad_weight: torch.Tensor          # [V, H]
    grad_logits: torch.Tensor          # [M, V] with respect to the unscaled logits


def fused_linear_scaled_ce_oracle(_input, weight, target, temperature=1.0, ignore_index=-100, grad_nll=None, grad_entropy=None,
                                  round_logits_to: Optional[torch.dtype] = None, round_dlogits_to: Optional[torch.dtype] = None,
                                  compute_dtype=torch.float64) -> ScaledCEResult:
    """s = (x . w^T) / T;  nll = lse(s) - s_y;  entropy = lse(s) - sum_j p_j s_j  (``:50-63`` of the reference file).
    Backward for upstream gradients g_nll, g_ent per token (``:66-93``):
      d s_j = g_nll (p_j - [j = y]) - g_ent p_j (log p_j + entropy),   d z = d s / T,
    masked on ignored tokens; grad_input = dz . w, grad_weight = dz^T . x."""
    x, w = _input.to(compute_dtype), weight.to(compute_dtype)
    m, v = x.shape[0], w.shape[0]
    live = target != ignore_index
    safe = target.masked_fill(~live, 0)
    s = _round(x @ w.T, round_logits_to) / temperature
    lse = torch.logsumexp(s, dim=-1)
    logp = s - lse[:, None]
    p = logp.exp()
    entropy = lse - (p * s).sum(dim=-1)
    nll = -logp.gather(-1, safe[:, None])[:, 0]
    mask = live.to(compute_dtype)
    ds = torch.zeros(m, v, dtype=compute_dtype)
    if grad_nll is not None:
        g = grad_nll.to(compute_dtype) * mask
        one_hot = torch.zeros(m, v, dtype=compute_dtype).scatter_(-1, safe[:, None], 1.0)
        ds += g[:, None] * (p - one_hot)
    if grad_entropy is not None:
        g = grad_entropy.to(compute_dtype) * mask
        ds += -g[:, None] * p * (logp + entropy[:, None])
    dz = _round(ds / temperature, round_dlogits_to)
    return ScaledCEResult(nll=nll * mask, entropy=entropy * mask, grad_input=dz @ w, grad_weight=dz.T @ x, grad_logits=dz)
