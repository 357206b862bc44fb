"""CPU oracle for fused linear cross-entropy (FLCE) forward + backward.

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA path: it may be
imported by the test-suite, by the smoke check and by the CPU-baseline leg of the
benchmark, never by the shipped package.

It restates, as closed-form tensor algebra on the host, what the reference computes
row by row on the GPU:

* per-row math (soft-capping, online max / sum-exp, label smoothing, z-loss, class
  weights, arg-max metrics, the logit gradient and its true-class entry):
  ``src/liger_kernel/ops/cross_entropy.py:97-336``
* batch-wide normalisers (count of non-ignored rows, sum of their class weights):
  ``src/liger_kernel/ops/fused_linear_cross_entropy.py:92-106``
* token scaling by the detached true-class probability:
  ``src/liger_kernel/ops/fused_linear_cross_entropy.py:123-150,199-218``
* projection of the logit gradient onto input / weight / bias:
  ``src/liger_kernel/ops/fused_linear_cross_entropy.py:225-265``
* reductions and output dtypes: ``src/liger_kernel/ops/fused_linear_cross_entropy.py:272-289``
* upstream-gradient scaling: ``src/liger_kernel/ops/fused_linear_cross_entropy.py:292-336``

Parity pin: ``tests/golden/*.npz`` hold outputs of the reference's own operator
(its Triton kernels executed by Triton's CPU interpreter) and of the torch
``Linear -> CrossEntropyLoss`` ground truth its tests use; ``tests/test_oracle.py``
checks this file against every one of them.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class OracleResult:
    loss: torch.Tensor  # scalar, or [N] for reduction="none"
    z_loss: torch.Tensor  # scalar, or [N]
    lse: torch.Tensor  # [N] log-sum-exp of the (soft-capped) logits; 0 on ignored rows
    token_accuracy: torch.Tensor  # scalar (mean over non-ignored), or [N]
    predicted_tokens: torch.Tensor  # [N] int64, -1 on ignored rows
    grad_input: Optional[torch.Tensor]  # [N, H]
    grad_weight: Optional[torch.Tensor]  # [V, H]
    grad_bias: Optional[torch.Tensor]  # [V] or None
    n_non_ignore: int


def _as(t, dtype):
    return None if t is None else t.detach().to("cpu").to(dtype)


def flce_oracle(
    _input: torch.Tensor,
    weight: torch.Tensor,
    target: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    ce_weight: Optional[torch.Tensor] = None,
    ignore_index: int = -100,
    lse_square_scale: float = 0.0,
    label_smoothing: float = 0.0,
    reduction: str = "mean",
    softcap: Optional[float] = None,
    use_token_scaling: bool = False,
    grad_output=None,
    compute_grads: bool = True,
    compute_dtype: torch.dtype = torch.float64,
    round_dlogits_to: Optional[torch.dtype] = None,
    row_chunk: int = 256,
    vocab_total: Optional[int] = None,
    n_non_ignore_override: Optional[int] = None,
    _given_logits: Optional[torch.Tensor] = None,
) -> OracleResult:
    """Closed-form FLCE.

    ``grad_output`` is the upstream gradient of the loss: a scalar for mean / sum
    (default 1) or an ``[N]`` vector for ``reduction="none"``.
    ``round_dlogits_to`` rounds the logit gradient to a storage dtype before the
    projections, as the reference does by writing it in place over its logits
    (``ops/cross_entropy.py:252``).  ``vocab_total`` lets label smoothing use a
    vocabulary larger than the local shard; ``n_non_ignore_override`` supplies a
    global count when rows are sharded across ranks.
    """
    assert reduction in ("mean", "sum", "none")
    cd = compute_dtype
    direct = _given_logits is not None  # stand-alone cross-entropy: logits are the input, no projection
    if direct:
        z_all = _as(_given_logits, cd)
        _input = torch.zeros(z_all.shape[0], 1)
        weight = torch.zeros(z_all.shape[1], 1)
    x = _as(_input, cd)
    w = _as(weight, cd)
    b = _as(bias, cd)
    cw = _as(ce_weight, cd)
    tgt = target.detach().to("cpu").to(torch.int64)
    n_rows, _ = x.shape
    vocab = w.shape[0]
    v_smooth = vocab if vocab_total is None else vocab_total
    alpha = float(label_smoothing)
    eps = alpha / v_smooth
    lam = float(lse_square_scale)

    valid = tgt != ignore_index
    n_valid = int(valid.sum()) if n_non_ignore_override is None else int(n_non_ignore_override)
    safe_t = torch.where(valid, tgt, torch.zeros_like(tgt))
    if cw is not None:
        w_y = cw[safe_t] * valid
        sum_w_valid = float(w_y.sum())
        sum_w = float(cw.sum())
    else:
        w_y = valid.to(cd)
        sum_w_valid = float(n_valid)
        sum_w = float(vocab)
    denom_loss = sum_w_valid if reduction == "mean" else 1.0
    denom_z = float(n_valid) if reduction == "mean" else 1.0

    if grad_output is None:
        go_rows = torch.ones(n_rows, dtype=cd)
    else:
        go = torch.as_tensor(grad_output).detach().to("cpu").to(cd)
        go_rows = go.expand(n_rows).clone() if go.dim() == 0 else go.reshape(n_rows)

    loss_rows = torch.zeros(n_rows, dtype=cd)
    z_rows = torch.zeros(n_rows, dtype=cd)
    lse_rows = torch.zeros(n_rows, dtype=cd)
    pred = torch.full((n_rows,), -1, dtype=torch.int64)
    correct = torch.zeros(n_rows, dtype=cd)
    dx = torch.zeros_like(x) if compute_grads else None
    dw = torch.zeros_like(w) if compute_grads else None
    db = torch.zeros(vocab, dtype=cd) if (compute_grads and b is not None) else None

    for r0 in range(0, n_rows, row_chunk):
        r1 = min(r0 + row_chunk, n_rows)
        xs = x[r0:r1]
        z = z_all[r0:r1] if direct else xs @ w.t()
        if b is not None:
            z = z + b
        if softcap is not None:
            th = torch.tanh(z / softcap)
            s = softcap * th
        else:
            th = None
            s = z
        v = valid[r0:r1]
        t = safe_t[r0:r1]
        m = s.max(dim=1).values
        d = torch.exp(s - m[:, None]).sum(dim=1)
        lse = m + torch.log(d)
        s_y = s.gather(1, t[:, None])[:, 0]
        p = torch.exp(s - lse[:, None])
        p_y = p.gather(1, t[:, None])[:, 0]
        wy = w_y[r0:r1]

        # ---- loss (ops/cross_entropy.py:296-326)
        row_loss = (lse - s_y) * (wy if cw is not None else 1.0)
        if alpha > 0:
            if cw is not None:
                smooth = (-eps * s * cw[None, :]).sum(dim=1) + eps * lse * sum_w
            else:
                smooth = (-eps * s).sum(dim=1) + alpha * lse
            row_loss = row_loss * (1 - alpha) + smooth
        row_z = lam * lse * lse
        if denom_loss != 0:
            row_loss = row_loss / denom_loss
        if denom_z != 0:
            row_z = row_z / denom_z
        row_total = row_loss + row_z
        scale_tok = p_y if use_token_scaling else torch.ones_like(p_y)
        vz = v.to(cd)
        loss_rows[r0:r1] = row_total * scale_tok * vz
        z_rows[r0:r1] = row_z * scale_tok * vz
        lse_rows[r0:r1] = lse * vz
        am = s.argmax(dim=1)  # torch returns the first index on ties, as the kernel does
        pred[r0:r1] = torch.where(v, am, torch.full_like(am, -1))
        correct[r0:r1] = ((am == t) & v).to(cd)

        if not compute_grads:
            continue
        # ---- gradient wrt the soft-capped logits (ops/cross_entropy.py:205-283)
        onehot = torch.zeros_like(p)
        onehot.scatter_(1, t[:, None], 1.0)
        if cw is None:
            g = p * (1 + 2 * lam * lse[:, None]) - eps - (1 - alpha) * onehot
            if reduction == "mean":
                g = g / n_valid if n_valid != 0 else g * 0
        else:
            ori = ((1 - alpha) * p - (1 - alpha) * onehot) * wy[:, None]
            smooth_g = eps * (-cw[None, :] + p * sum_w)
            zg = 2 * lam * lse[:, None] * p
            if reduction == "mean":
                ori = ori / sum_w_valid
                smooth_g = smooth_g / sum_w_valid
                zg = zg / n_valid
            g = ori + smooth_g + zg
        if th is not None:
            g = g * (1 - th * th)
        g = g * (scale_tok * vz * go_rows[r0:r1])[:, None]
        if round_dlogits_to is not None:
            g = g.to(round_dlogits_to).to(cd)
        if direct:
            if r0 == 0:
                dx = torch.zeros_like(z_all)
            dx[r0:r1] = g
            continue
        dx[r0:r1] = g @ w
        dw += g.t() @ xs
        if db is not None:
            db += g.sum(dim=0)

    if reduction == "none":
        loss, zl, acc = loss_rows, z_rows, correct
    else:
        loss, zl = loss_rows.sum(), z_rows.sum()
        acc = correct.sum() / n_valid if n_valid != 0 else correct.sum() * float("nan")
    return OracleResult(loss, zl, lse_rows, acc, pred, dx, dw, db, n_valid)


def ce_oracle(logits, target, weight=None, ignore_index=-100, lse_square_scale=0.0, label_smoothing=0.0, reduction="mean",
              softcap=None, grad_output=None, compute_dtype=torch.float64) -> OracleResult:
    """Stand-alone cross-entropy on given logits (``src/liger_kernel/ops/cross_entropy.py:97-336, 351-502``):
    same closed form as above without the linear layer; ``grad_input`` is the gradient with respect to the logits."""
    return flce_oracle(None, None, target, ce_weight=weight, ignore_index=ignore_index, lse_square_scale=lse_square_scale,
                       label_smoothing=label_smoothing, reduction=reduction, softcap=softcap, grad_output=grad_output,
                       compute_dtype=compute_dtype, _given_logits=logits)


def torch_linear_ce_reference(
    _input,
    weight,
    target,
    bias=None,
    ce_weight=None,
    ignore_index=-100,
    lse_square_scale=0.0,
    label_smoothing=0.0,
    reduction="mean",
    softcap=None,
    dtype=torch.float32,
):
    """``Linear -> float -> soft-cap -> F.cross_entropy + z-loss`` with torch autograd.

    This is the ground truth of the reference's FLCE tests
    (``test/transformers/test_fused_linear_cross_entropy.py:22-67`` on top of
    ``test/transformers/test_cross_entropy.py:22-78``), written out again; it is
    what the CPU baseline of the benchmark times on the host cores.
    Returns ``(loss, z_loss, grad_input, grad_weight, grad_bias)``.
    """
    x = _input.detach().to("cpu").to(dtype).requires_grad_(True)
    w = weight.detach().to("cpu").to(dtype).requires_grad_(True)
    b = None if bias is None else bias.detach().to("cpu").to(dtype).requires_grad_(True)
    cw = None if ce_weight is None else ce_weight.detach().to("cpu").to(dtype)
    t = target.detach().to("cpu").to(torch.int64)
    logits = torch.nn.functional.linear(x, w, b).float() if dtype != torch.float64 else torch.nn.functional.linear(x, w, b)
    if softcap is not None:
        logits = softcap * torch.tanh(logits / softcap)
    ce = torch.nn.functional.cross_entropy(
        logits, t, weight=cw, ignore_index=ignore_index, label_smoothing=label_smoothing, reduction=reduction
    )
    lse = torch.logsumexp(logits, dim=-1)
    mask = t != ignore_index
    z_rows = torch.where(mask, lse_square_scale * lse * lse, torch.zeros_like(lse))
    if reduction == "mean":
        z = z_rows.sum() / mask.sum()
    elif reduction == "sum":
        z = z_rows.sum()
    else:
        z = z_rows
    total = ce + z
    if reduction == "none":
        total.sum().backward()
    else:
        total.backward()
    return total.detach(), z.detach(), x.grad, w.grad, None if b is None else b.grad
