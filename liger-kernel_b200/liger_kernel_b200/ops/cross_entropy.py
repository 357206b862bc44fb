"""Stand-alone cross-entropy on materialised logits, host side.

Call surface of the reference's ``src/liger_kernel/ops/cross_entropy.py`` (``cross_entropy_forward`` /
``cross_entropy_backward`` / ``LigerCrossEntropyFunction``, ``:351-606``) on the CUDA kernels of ``libflce_b200.so``.

Two forms.  When the logits require a gradient (and the caller is recording), forward forms the gradient in the same
launch, for an upstream gradient of 1, and backward only folds the real upstream gradient in, exactly the reference's
arrangement (``:428-466``, ``:477-502``); each row stays in the shared memory of a thread-block cluster between the two passes,
so HBM sees 2 x BT x V elements.  With ``INPLACE_GRADIENT`` (default, and what the reference does) the gradient replaces the
logits in forward.  Otherwise, and for rows the cluster form cannot hold (longer than 1.6 MB, or not 16-byte aligned),
forward reads the logits once and leaves them untouched and backward reads them again and writes the gradient (3 x BT x V).
``MODE = "two_pass"`` (``LIGER_B200_CE_MODE``) forces the second form.  There is no host synchronisation in either: a scalar
upstream gradient of 1 is recognised on the device, and out-of-range targets are not reported (they simply match no class)
unless ``LIGER_B200_CHECK_TARGETS=1`` asks for the reference's assertion.
"""

from __future__ import annotations

import ctypes as C
import os
import threading
from typing import Optional

import torch

from .. import _lib
from .._lib import CeProblem, check, lib
from . import fused_linear_cross_entropy as _fl
from .fused_linear_cross_entropy import _DTYPES, _REDUCTIONS, _as_forward_out, _ptr

# write the logit gradient over the logits' own storage (as the reference does, to avoid a second [BT, V] buffer);
# set to False to get a fresh tensor and keep the logits intact
INPLACE_GRADIENT = True
# "auto": gradient formed in forward whenever the logits require one and the rows qualify; "two_pass": never
MODE = os.environ.get("LIGER_B200_CE_MODE", "auto")
_grad_mode = threading.local()


class _CePrepared:
    def __init__(self, _input, target, weight, ignore_index, lse_square_scale, label_smoothing, reduction, softcap):
        _fl._require_cuda(_input)
        if _input.dim() != 2:
            raise ValueError(f"expected logits [BT, V], got {tuple(_input.shape)}")
        if target.dim() != 1 or target.shape[0] != _input.shape[0]:
            raise ValueError(f"target must be [BT]={_input.shape[0]}, got {tuple(target.shape)}")
        if _input.dtype not in _DTYPES:
            raise TypeError(f"unsupported dtype {_input.dtype}")
        if reduction not in _REDUCTIONS:
            raise ValueError(f"reduction must be 'mean', 'sum' or 'none'. Got: {reduction}")
        if weight is not None:
            assert weight.shape[0] == _input.shape[1], f"If given, weight has to be a Tensor of size V. Got: {weight.shape}"
            assert torch.is_floating_point(weight), f"If given, weight has to be a Tensor of floating point dtype. Got: {weight.dtype}"
        self.device = _input.device
        self.dtype = _input.dtype
        self.n_rows, self.vocab = _input.shape
        self.reduction = reduction
        self.logits = _input.detach() if _input.stride(-1) == 1 else _input.detach().contiguous()
        self.target = target.detach().to(device=self.device, dtype=torch.int64).contiguous()
        self.weight = None if weight is None else weight.detach().to(device=self.device, dtype=torch.float32).contiguous()
        p = CeProblem()
        p.n_rows, p.vocab, p.ld = self.n_rows, self.vocab, self.logits.stride(0)
        p.dtype, p.reduction = _DTYPES[self.dtype], _REDUCTIONS[reduction]
        p.ignore_index = int(ignore_index)
        p.label_smoothing, p.lse_square_scale = float(label_smoothing), float(lse_square_scale)
        p.softcap = 0.0 if softcap is None else float(softcap)
        p.logits, p.target = self.logits.data_ptr(), self.target.data_ptr()
        p.ce_weight = None if self.weight is None else self.weight.data_ptr()
        self.problem = p


def _fused_form_applies(prep) -> bool:
    """Rows the cluster kernel can hold (mirrors the checks of ``flce_b200_ce_forward_backward``)."""
    esize = prep.logits.element_size()
    row_bytes = prep.vocab * esize
    return (MODE != "two_pass" and row_bytes % 16 == 0 and row_bytes <= 8 * 200 * 1024
            and prep.logits.data_ptr() % 16 == 0 and (prep.logits.stride(0) * esize) % 16 == 0)


def cross_entropy_forward(_input, target, weight, ignore_index, lse_square_scale, label_smoothing, reduction, softcap,
                          return_z_loss, return_token_accuracy=False, return_predicted_tokens=False, with_gradient=False,
                          inplace: Optional[bool] = None):
    """Returns ``(loss, z_loss, token_accuracy, predicted_tokens, saved)``; ``saved`` feeds ``cross_entropy_backward``.
    loss and z_loss come back in the logits' dtype, as in the reference (``ops/cross_entropy.py:378-380``).
    ``with_gradient`` asks for the gradient to be formed in the same launch where the rows allow it (``saved`` then carries
    the gradient, which with ``inplace`` has replaced the logits)."""
    assert isinstance(return_z_loss, bool), f"return_z_loss must be True or False. Got: {return_z_loss}"
    assert isinstance(return_token_accuracy, bool), f"return_token_accuracy must be True or False. Got: {return_token_accuracy}"
    assert isinstance(return_predicted_tokens, bool), f"return_predicted_tokens must be True or False. Got: {return_predicted_tokens}"
    prep = _CePrepared(_input, target, weight, ignore_index, lse_square_scale, label_smoothing, reduction, softcap)
    n, dev = prep.n_rows, prep.device
    f32 = dict(dtype=torch.float32, device=dev)
    out = dict(lse=torch.empty(n, **f32), target_prob=torch.empty(n, **f32), loss_rows=torch.empty(n, **f32),
               z_loss_rows=torch.empty(n, **f32), correct_rows=torch.empty(n, **f32),
               predicted_tokens=torch.empty(n, dtype=torch.int64, device=dev), scalars=torch.empty(4, **f32))
    norm = torch.empty(4, **f32)
    rowstats = torch.empty((_lib.ROWSTAT_PLANES, n), **f32)
    fo = _as_forward_out(out)
    grad = None
    if with_gradient and _fused_form_applies(prep):
        inplace = INPLACE_GRADIENT if inplace is None else inplace
        grad = prep.logits if inplace else torch.empty_like(prep.logits)
    with _fl._device_guard(dev):
        if grad is not None:
            check(lib.flce_b200_ce_forward_backward(C.byref(prep.problem), _ptr(norm), _ptr(rowstats), C.byref(fo), _ptr(grad),
                                                    grad.stride(0), _fl._stream(dev)))
        else:
            check(lib.flce_b200_ce_forward(C.byref(prep.problem), _ptr(norm), _ptr(rowstats), C.byref(fo), _fl._stream(dev)))
    if _fl.CHECK_TARGETS:      # the reference's assertion (ops/cross_entropy.py:389-392), at the price of a host synchronisation
        _fl._raise_on_bad_targets(norm, prep.vocab)
    if reduction == "none":
        loss = out["loss_rows"].to(prep.dtype)
        z_loss = out["z_loss_rows"].to(prep.dtype) if return_z_loss else None
        token_accuracy = out["correct_rows"] if return_token_accuracy else None
    else:
        loss = out["scalars"][0].to(prep.dtype)
        z_loss = out["scalars"][1].to(prep.dtype) if return_z_loss else None
        token_accuracy = out["scalars"][2] if return_token_accuracy else None
    predicted_tokens = out["predicted_tokens"] if return_predicted_tokens else None
    return loss, z_loss, token_accuracy, predicted_tokens, (prep, out["lse"], norm, grad)


def cross_entropy_backward(saved, grad_output, inplace: Optional[bool] = None):
    """Gradient with respect to the logits, ``grad_output`` (scalar, or per row for ``reduction="none"``) folded in."""
    prep, lse, norm, formed = saved
    dev = prep.device
    go = grad_output.detach().to(device=dev, dtype=torch.float32).contiguous().reshape(-1)
    if go.numel() not in (1, prep.n_rows):
        raise ValueError(f"grad_output must have 1 or {prep.n_rows} elements, got {go.numel()}")
    per_row = int(go.numel() == prep.n_rows and prep.reduction == "none")
    if formed is not None:
        # formed in forward for an upstream gradient of 1 (the reference's cross_entropy_backward, :477-502)
        with _fl._device_guard(dev):
            check(lib.flce_b200_ce_scale_gradient(_ptr(formed), formed.stride(0), prep.n_rows, prep.vocab, _DTYPES[prep.dtype],
                                                  _ptr(go), per_row, _fl._stream(dev)))
        return formed
    inplace = INPLACE_GRADIENT if inplace is None else inplace
    grad = prep.logits if inplace else torch.empty_like(prep.logits)
    scratch = torch.empty(3 * prep.n_rows, dtype=torch.float32, device=dev)
    with _fl._device_guard(dev):
        check(lib.flce_b200_ce_backward(C.byref(prep.problem), _ptr(lse), _ptr(norm), _ptr(go), per_row, _ptr(grad),
                                        grad.stride(0), _ptr(scratch), _fl._stream(dev)))
    return grad


class LigerCrossEntropyFunction(torch.autograd.Function):
    """Drop-in for the reference class of the same name (``ops/cross_entropy.py:504-606``): 11 arguments, 4-tuple result."""

    @classmethod
    def apply(cls, *args, **kwargs):
        # grad mode is always off inside forward(): note here whether the caller is recording, so that an evaluation
        # loop under torch.no_grad() neither pays for a gradient nor loses its logits to one
        _grad_mode.enabled = torch.is_grad_enabled()
        try:
            return super().apply(*args, **kwargs)
        finally:
            _grad_mode.enabled = True

    @staticmethod
    def forward(ctx, _input, target, weight, ignore_index=-100, lse_square_scale=0.0, label_smoothing=0.0,
                reduction="mean", softcap=None, return_z_loss=False, return_token_accuracy=False,
                return_predicted_tokens=False):
        recording = getattr(_grad_mode, "enabled", True) and ctx.needs_input_grad[0]
        loss, z_loss, token_accuracy, predicted_tokens, saved = cross_entropy_forward(
            _input, target, weight, ignore_index, lse_square_scale, label_smoothing, reduction, softcap, return_z_loss,
            return_token_accuracy, return_predicted_tokens, with_gradient=bool(recording))
        ctx.ce_saved = saved
        ctx.ce_formed_in_forward = saved[3] is not None
        ctx.in_shape, ctx.in_dtype = _input.shape, _input.dtype
        nondiff = [t for t in (z_loss, token_accuracy, predicted_tokens) if t is not None]
        if nondiff:
            ctx.mark_non_differentiable(*nondiff)
        return loss, z_loss, token_accuracy, predicted_tokens

    @staticmethod
    def backward(ctx, grad_output, grad_output2=None, grad_output3=None, grad_output4=None):
        if getattr(ctx, "ce_logits_overwritten", False):
            raise RuntimeError(
                "the logits were overwritten by the gradient of the first backward (INPLACE_GRADIENT); set "
                "liger_kernel_b200.ops.cross_entropy.INPLACE_GRADIENT = False to run backward more than once")
        if ctx.ce_formed_in_forward and getattr(ctx, "ce_gradient_used", False):
            raise RuntimeError(
                "the gradient formed in forward was overwritten when the first backward folded its upstream gradient in; set "
                "liger_kernel_b200.ops.cross_entropy.MODE = 'two_pass' and INPLACE_GRADIENT = False to run backward more than once")
        saved = ctx.ce_saved
        grad = cross_entropy_backward(saved, grad_output)
        ctx.ce_logits_overwritten = INPLACE_GRADIENT
        ctx.ce_gradient_used = True
        if ctx.ce_logits_overwritten or ctx.ce_formed_in_forward:
            # no second backward is possible: let go of the buffers, so that the gradient returned here is the only
            # reference to its tensor and a leaf's .grad can take it as it is instead of copying BT x V elements
            ctx.ce_saved = None
            saved[0].logits = None
        return (grad,) + (None,) * 10
