"""Fused linear generalised Jensen-Shannon divergence (distillation loss on two language-model heads), host side.

Call surface of the reference's ``src/liger_kernel/ops/fused_linear_jsd.py`` (``fused_linear_jsd_forward`` ``:23-157``,
``fused_linear_jsd_backward`` ``:160-192``, ``LigerFusedLinearJSDFunction`` ``:195-265``).  Like the reference, the
gradients are formed in forward (the loss is the last node of the graph) over token chunks, so no ``[BT, V]`` tensor
outlives a chunk; ``backward`` only scales them by the upstream gradient.

Per chunk: student and teacher logits by two tcgen05 GEMMs into slabs of the operands' dtype, one row kernel that reads both slabs
(log-normalisers, loss, chain rule through ``log_softmax`` and the temperature) and leaves the student's logit gradient
in the student's slab, then ``grad_input = dZ . W`` and ``grad_weight += dZ^T . X`` (fp32 accumulator across chunks).

Differences a caller can observe: no host synchronisation (the reference reads the count of non-ignored labels with
``.item()``); ``grad_weight`` is always accumulated in fp32 (``accum_dtype`` is accepted and has nothing left to select); fp32
operands run on the tensor cores as sums of bf16 term products (see ``_chunked.py``).
"""

from __future__ import annotations

from typing import Optional

import torch

from .._lib import check
from . import _chunked as ck
from . import fused_linear_cross_entropy as _fl
from .fused_linear_cross_entropy import _DTYPES, _ptr, scale_gradient_


def fused_linear_jsd_forward(student_input, student_weight, teacher_input, teacher_weight, shift_labels, jsd_beta,
                             ignore_index, has_label, temperature, accum_dtype=None, weight_requires_grad=None,
                             input_requires_grad=True):
    """Returns ``(loss, grad_input, grad_weight)``; ``grad_weight`` is None when the student head needs no gradient
    (``weight_requires_grad``, by default ``student_weight.requires_grad`` as in the reference) and ``grad_input`` is None
    when ``input_requires_grad`` is False (an evaluation pass then costs the two logits GEMMs and the row kernel only)."""
    for t in (student_input, student_weight, teacher_input, teacher_weight):
        _fl._require_cuda(t)
    if student_input.dim() != 2 or teacher_input.dim() != 2 or student_weight.dim() != 2 or teacher_weight.dim() != 2:
        raise ValueError("expected student_input [BT, H], student_weight [V, H], teacher_input [BT, H'], teacher_weight [V, H']")
    n_rows, hs = student_input.shape
    vocab = student_weight.shape[0]
    if teacher_input.shape[0] != n_rows or teacher_weight.shape[0] != vocab:
        raise ValueError(f"student and teacher disagree on BT or V: {tuple(student_input.shape)} {tuple(student_weight.shape)} "
                         f"vs {tuple(teacher_input.shape)} {tuple(teacher_weight.shape)}")
    if student_weight.shape[1] != hs or teacher_weight.shape[1] != teacher_input.shape[1]:
        raise ValueError("hidden sizes of inputs and weights do not match")
    dtype = student_input.dtype
    if not (student_weight.dtype == teacher_input.dtype == teacher_weight.dtype == dtype):
        raise TypeError("student and teacher tensors must share one dtype")
    if not 0.0 <= float(jsd_beta) <= 1.0:
        raise ValueError(f"jsd_beta must be in [0, 1]. Got: {jsd_beta}")
    dev = student_input.device
    lib = ck._lib_handle()
    need_weight = bool(student_weight.requires_grad if weight_requires_grad is None else weight_requires_grad)

    student = ck.Head(student_input, student_weight, need_grads=True)
    teacher = ck.Head(teacher_input, teacher_weight, need_grads=False)
    labels = None
    count = None
    if has_label:
        labels = shift_labels.detach().to(device=dev, dtype=torch.int64).contiguous()
        count = (labels != ignore_index).sum().to(torch.float32).reshape(1)      # stays on the device
    chunk_rows, n_chunks = ck.plan_chunks(n_rows, student.slab_bytes_per_row() + teacher.slab_bytes_per_row())
    slab_s, slab_t = student.new_slab(chunk_rows), teacher.new_slab(chunk_rows)
    need_input = bool(input_requires_grad)
    grad_input = student.new_grad_input() if need_input else None
    grad_weight32 = student.new_grad_weight() if need_weight else None
    loss_rows = torch.empty(n_rows, dtype=torch.float32, device=dev)
    with _fl._device_guard(dev):
        for c in range(n_chunks):
            r0 = c * chunk_rows
            rows = min(chunk_rows, n_rows - r0)
            student.logits(r0, rows, slab_s)
            teacher.logits(r0, rows, slab_t)
            check(lib.flce_b200_jsd_rows(
                _ptr(slab_s), slab_s.stride(0), _ptr(slab_t), slab_t.stride(0), _DTYPES[dtype], rows, vocab,
                None if labels is None else _ptr(labels[r0:r0 + rows]), int(ignore_index), float(jsd_beta), float(temperature),
                _ptr(count), float(n_rows), _ptr(loss_rows[r0:r0 + rows]), _fl._stream(dev)))
            if need_input or need_weight:
                student.project(slab_s, r0, rows, grad_input[r0:r0 + rows] if need_input else None, grad_weight32)
    loss = loss_rows.sum()
    return loss, student.finish_grad_input(grad_input), student.finish_grad_weight(grad_weight32)


def fused_linear_jsd_backward(grad_output, grad_input, grad_weight):
    """``grad *= grad_output`` unless the upstream gradient is exactly 1 (tested on the device)."""
    present = grad_input if grad_input is not None else grad_weight
    if present is None:
        return None, None
    go = grad_output.detach().to(device=present.device, dtype=torch.float32).reshape(1)
    grad_input = scale_gradient_(grad_input, go)
    grad_weight = scale_gradient_(grad_weight, go)
    return grad_input, grad_weight


class LigerFusedLinearJSDFunction(torch.autograd.Function):
    """Drop-in for the reference class of the same name (``ops/fused_linear_jsd.py:195-265``): 9 arguments, scalar loss."""

    @staticmethod
    def forward(ctx, student_input: torch.Tensor, student_weight: torch.Tensor, teacher_input: torch.Tensor,
                teacher_weight: torch.Tensor, shift_labels: Optional[torch.Tensor] = None, jsd_beta: float = 0.5,
                ignore_index: int = -100, temperature: float = 1.0, accum_dtype: Optional[torch.dtype] = None):
        has_label = False
        if shift_labels is not None:
            assert shift_labels.shape == (teacher_input.shape[0],), (
                f"the shape of shift_labels must be (BT,). Got: {shift_labels.shape}"
            )
            shift_labels = shift_labels.contiguous()
            has_label = True
        in_dtypes = (student_input.dtype, student_weight.dtype)
        if torch.is_autocast_enabled("cuda") and student_input.device.type == "cuda":
            dt = torch.get_autocast_dtype("cuda")
            student_input, student_weight = student_input.to(dt), student_weight.to(dt)
            teacher_input, teacher_weight = teacher_input.to(dt), teacher_weight.to(dt)
        loss, grad_input, grad_weight = fused_linear_jsd_forward(
            student_input, student_weight, teacher_input, teacher_weight, shift_labels, jsd_beta, ignore_index, has_label,
            temperature, accum_dtype, weight_requires_grad=ctx.needs_input_grad[1], input_requires_grad=ctx.needs_input_grad[0])
        ctx.jsd_grads = (grad_input, grad_weight)
        ctx.jsd_handed_off = False
        ctx.jsd_in_dtypes = in_dtypes
        return loss

    @staticmethod
    def backward(ctx, grad_output):
        grad_input, grad_weight = ctx.jsd_grads
        if ctx.jsd_handed_off:
            raise RuntimeError("the gradients of this fused linear JSD call were already handed off by an earlier backward")
        ctx.jsd_handed_off = True
        ctx.jsd_grads = (None, None)
        grad_input, grad_weight = fused_linear_jsd_backward(grad_output, grad_input, grad_weight)
        dx, dw = ctx.jsd_in_dtypes
        grad_input = None if grad_input is None else grad_input.to(dx)
        grad_weight = None if grad_weight is None else grad_weight.to(dw)
        return (grad_input, grad_weight) + (None,) * 7
