"""Final RMSNorm + lm_head + cross-entropy as one operator.

The reference runs the decoder's last norm as a kernel pair of its own (``src/liger_kernel/ops/rms_norm.py:59-235``) and hands
its output to the fused head (``src/liger_kernel/transformers/model/llama.py:95-98``).  Here the norm rides on the two row moves
the fused path makes anyway: the gather that puts the rows that matter in front of the tensor-core sweeps normalises them on
the way (``flce_b200_compact_rows_rmsnorm``), and the scatter that brings grad_input back to token order applies the norm's
backward on the way (``flce_b200_rmsnorm_scatter_backward``).  Rows whose target is ``ignore_index`` are normalised but take
no part in any GEMM; their gradient is exact zero.

Scope: bf16 / fp16 hidden states, hidden size a multiple of 8 and at most 16384, casting modes "llama" and "gemma"
(``ops/rms_norm.py:52-54``), ``reduction`` "mean" or "sum" whenever a gradient is wanted (the gradients are formed in forward,
as in the default mode of the fused head).  Everything else raises ``NotImplementedError`` rather than being ignored.
"""

from __future__ import annotations

import threading

import torch

from . import fused_linear_cross_entropy as _fl
from .fused_linear_cross_entropy import (_Prepared, _autocast_operands, _raise_on_bad_targets, _results_to_token_order,
                                         flce_forward_device, flce_single_sweep_device, scale_gradient_)

_grad_mode = threading.local()


class LigerFusedRMSNormLinearCrossEntropyFunction(torch.autograd.Function):
    """``loss(lm_head(rms_norm(hidden)))``.  Arguments: hidden ``[BT, H]`` (before the norm), norm_weight ``[H]``, weight
    ``[V, H]``, target ``[BT]``, then ``eps``, ``offset``, ``casting_mode`` of the norm and the keyword set of
    ``LigerFusedLinearCrossEntropyFunction``.  Returns ``(loss, z_loss, token_accuracy, predicted_tokens)``; gradients flow to
    hidden, norm_weight, weight and bias."""

    @classmethod
    def apply(cls, *args, **kwargs):
        _grad_mode.enabled = torch.is_grad_enabled()
        try:
            return super().apply(*args, **kwargs)
        finally:
            _grad_mode.enabled = True

    @staticmethod
    def forward(ctx, hidden, norm_weight, weight, target, eps=1e-6, offset=0.0, casting_mode="llama", bias=None, ce_weight=None,
                ignore_index=-100, lse_square_scale=0.0, label_smoothing=0.0, reduction="mean", softcap=None,
                return_z_loss: bool = False, use_token_scaling: bool = False, return_token_accuracy: bool = False,
                return_predicted_tokens: bool = False):
        ctx.in_dtypes = (hidden.dtype, norm_weight.dtype, weight.dtype, None if bias is None else bias.dtype)
        x, w, b = _autocast_operands(hidden, weight, bias)
        recording = getattr(_grad_mode, "enabled", True)
        need_h, need_g, need_w = (recording and ctx.needs_input_grad[i] for i in (0, 1, 2))
        need_b = recording and bias is not None and ctx.needs_input_grad[7]
        wants = need_h or need_g or need_w or need_b
        if wants and not _fl._use_single_sweep(reduction, (True, True), x.dtype):
            raise NotImplementedError("the fused RMSNorm head forms its gradients in forward: reduction must be 'mean' or 'sum' "
                                      "and the operands 16-bit (LIGER_B200_FLCE_MODE must not be 'recompute')")
        prep = _Prepared(x, w, target, b, ce_weight, ignore_index, lse_square_scale, label_smoothing, reduction, softcap,
                         use_token_scaling, want_argmax=return_token_accuracy or return_predicted_tokens, allow_compact=True,
                         rms_norm=dict(weight=norm_weight, eps=eps, offset=offset, casting_mode=casting_mode))
        ctx.stored = None
        if wants:
            out, norm, gy, gw, gb = flce_single_sweep_device(prep, need_h or need_g, need_w, need_b)
            gh = gg = None
            if gy is not None:
                gh, gg = prep.rmsnorm_backward(gy)
            ctx.stored = (gh if need_h else None, gg if need_g else None, gw, gb)
        else:
            out, norm, _rowstats = flce_forward_device(prep)
        out = _results_to_token_order(prep, out)
        if _fl.CHECK_TARGETS:
            _raise_on_bad_targets(norm, prep.vocab)
        if reduction == "none":
            loss = out["loss_rows"]
            z_loss = out["z_loss_rows"].to(prep.dtype) if return_z_loss else None
            token_accuracy = out["correct_rows"] if return_token_accuracy else None
        else:
            loss = out["scalars"][0]
            z_loss = out["scalars"][1].to(prep.dtype) if return_z_loss else None
            token_accuracy = out["scalars"][2] if return_token_accuracy else None
        predicted_tokens = out["predicted_tokens"] if return_predicted_tokens else None
        nondiff = [t for t in (z_loss, token_accuracy, predicted_tokens) if t is not None]
        if nondiff:
            ctx.mark_non_differentiable(*nondiff)
        return loss, z_loss, token_accuracy, predicted_tokens

    @staticmethod
    def backward(ctx, grad_output, grad_output2=None, grad_output3=None, grad_output4=None):
        if ctx.stored is None:
            raise RuntimeError("the gradients of the fused RMSNorm head are formed in forward and handed out once; run forward "
                               "again for another backward")
        gh, gg, gw, gb = ctx.stored
        ctx.stored = None
        dev = next(t for t in (gh, gg, gw, gb) if t is not None).device
        go = grad_output.detach().to(device=dev, dtype=torch.float32).reshape(1)
        gh, gg, gw, gb = (scale_gradient_(t, go) for t in (gh, gg, gw, gb))
        dh, dg, dw, db = ctx.in_dtypes
        cast = lambda t, d: None if t is None else t.to(d)   # noqa: E731
        return (cast(gh, dh), cast(gg, dg), cast(gw, dw), None, None, None, None, cast(gb, db)) + (None,) * 10


def liger_fused_rmsnorm_linear_cross_entropy(hidden, norm_weight, weight, target, eps=1e-6, offset=0.0, casting_mode="llama",
                                             bias=None, ce_weight=None, ignore_index=-100, lse_square_scale=0.0,
                                             label_smoothing=0.0, reduction="mean", softcap=None, return_z_loss=False,
                                             use_token_scaling=False, return_token_accuracy=False,
                                             return_predicted_tokens=False):
    """Functional form: the loss alone, or a ``CrossEntropyOutput`` when any of the ``return_*`` flags is set (the convention of
    ``liger_fused_linear_cross_entropy``)."""
    from ..transformers.functional import CrossEntropyOutput

    loss, z_loss, token_accuracy, predicted_tokens = LigerFusedRMSNormLinearCrossEntropyFunction.apply(
        hidden, norm_weight, weight, target, eps, offset, casting_mode, bias, ce_weight, ignore_index, lse_square_scale,
        label_smoothing, reduction, softcap, return_z_loss, use_token_scaling, return_token_accuracy, return_predicted_tokens)
    if not (return_z_loss or return_token_accuracy or return_predicted_tokens):
        return loss
    return CrossEntropyOutput(loss=loss, z_loss=z_loss, token_accuracy=token_accuracy, predicted_tokens=predicted_tokens)
