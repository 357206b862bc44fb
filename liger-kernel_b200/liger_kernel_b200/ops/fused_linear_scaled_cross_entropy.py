"""Fused linear scaled cross-entropy: per-token negative log-likelihood and entropy of ``softmax(x . W^T / T)`` without
keeping the ``[M, V]`` logits (the policy-gradient head of RL fine-tuning), host side.

Call surface of the reference's ``src/liger_kernel/ops/fused_linear_scaled_cross_entropy.py``
(``LigerFusedLinearScaledCrossEntropyFunction.apply`` ``:163-199``; math of ``:50-93``).

Two forms (``MODE``).  ``"fused"`` (16-bit operands, default): the two tensor-core sweeps of the main path with scaled
cross-entropy epilogues -- sweep 1 keeps max / sum-exp / sum exp*s per (row, tile), nothing of size M x V is written;
backward recomputes the logits per vocabulary slab, forms the logit gradient in the epilogue and projects it
(``flce_b200_sce_forward`` / ``flce_b200_sce_backward``).  ``"chunked"`` (and fp32 operands): per token chunk, logits
by one tcgen05 GEMM into a slab of the operands' dtype and one row kernel (online max / sum-exp / sum of p.s in a single read).
Backward: the upstream gradients of both outputs arrive per token, so the chunk's logits are recomputed (as the
reference's device-independent path does), turned into the logit gradient in place, and projected twice
(``grad_input = dZ . W``, ``grad_weight += dZ^T . X`` with an fp32 accumulator across chunks).

Differences a caller can observe: targets are not range-checked on the host (that would synchronise; a target that is
neither ``ignore_index`` nor a class id contributes ``nll = lse``); fp32 operands run on the tensor cores as sums of
bf16 term products (see ``_chunked.py``); ``m_tiles_per_cluster`` is accepted and validated but selects nothing here.
"""

from __future__ import annotations

import ctypes as C
import math
import os

import torch

from .. import _lib
from .._lib import SceProblem, check
from . import _chunked as ck
from . import fused_linear_cross_entropy as _fl
from .fused_linear_cross_entropy import _DTYPES, _ptr


# "fused": 16-bit operands run on the two tensor-core sweeps of the main path with scaled cross-entropy epilogues (no logits
# slab in forward, vocabulary slabs of the logit gradient in backward); "chunked": the token-chunk loop over a logits slab.
# fp32 operands always take the chunked form.
MODE = os.environ.get("LIGER_B200_SCE_MODE", "fused")
SLAB_BUDGET_BYTES = 1 << 30


def _validate_temperature(temperature):
    if isinstance(temperature, bool) or not isinstance(temperature, (int, float)):
        raise TypeError("temperature must be a real number")
    if not math.isfinite(temperature) or temperature <= 0:
        raise ValueError("temperature must be finite and > 0")


def _validate_inputs(_input, weight, target):
    if _input.ndim != 2 or weight.ndim != 2 or target.ndim != 1:
        raise ValueError("expected input[M,H], weight[V,H], and target[M]")
    if _input.shape[0] != target.shape[0] or _input.shape[1] != weight.shape[1]:
        raise ValueError(
            f"input {tuple(_input.shape)}, weight {tuple(weight.shape)} and target "
            f"{tuple(target.shape)} shapes are incompatible"
        )
    if _input.shape[0] == 0 or _input.shape[1] == 0 or weight.shape[0] == 0:
        raise ValueError("input, hidden, and vocabulary dimensions must be non-empty")
    if _input.device != weight.device or _input.device != target.device:
        raise ValueError("input, weight, and target must be on the same device")
    if _input.dtype != weight.dtype or not torch.is_floating_point(_input):
        raise TypeError("input and weight must have the same floating-point dtype")
    if target.dtype != torch.int64:
        raise TypeError("target must be an int64 tensor")


def _fused_problem(x, w, target, temperature, ignore_index):
    p = SceProblem()
    p.n_rows, p.hidden, p.vocab = x.shape[0], x.shape[1], w.shape[0]
    p.ld_x, p.ld_w = x.stride(0), w.stride(0)
    p.dtype = _DTYPES[x.dtype]
    p.ignore_index = int(ignore_index)
    p.temperature = float(temperature)
    p.x, p.w, p.target = x.data_ptr(), w.data_ptr(), target.data_ptr()
    return p


def _workspace(n_bytes, device):
    return torch.empty(max(int(n_bytes), 256), dtype=torch.uint8, device=device)


def _fused_forward(ctx, hidden_states, vocab_weights, input_ids, temperature, ignore_index, return_entropy):
    dev, dtype = hidden_states.device, hidden_states.dtype
    lib = ck._lib_handle()
    x, w = _fl._pad_hidden(hidden_states.detach()), _fl._pad_hidden(vocab_weights.detach())
    target = input_ids.detach().contiguous()
    prob = _fused_problem(x, w, target, temperature, ignore_index)
    n_rows = x.shape[0]
    nll = torch.empty(n_rows, dtype=torch.float32, device=dev)
    entropy = torch.empty(n_rows, dtype=torch.float32, device=dev)
    lse = torch.empty(n_rows, dtype=torch.float32, device=dev)
    with _fl._device_guard(dev):
        ws = _workspace(lib.flce_b200_sce_workspace_bytes(C.byref(prob), _lib.PHASE_FORWARD, 0), dev)
        check(lib.flce_b200_sce_forward(C.byref(prob), _ptr(nll), _ptr(entropy), _ptr(lse), _ptr(ws), ws.numel(), _fl._stream(dev)))
    ctx.sce = ("fused", x, w, target, lse, entropy, float(temperature), int(ignore_index), hidden_states.shape[1])
    if return_entropy:
        return nll, entropy.to(dtype)
    return nll


def _fused_backward(ctx, grad_nll, grad_entropy):
    _, x, w, target, lse, entropy, temperature, ignore_index, hidden = ctx.sce
    need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
    dev, dtype = x.device, x.dtype
    lib = ck._lib_handle()
    n_rows, h8 = x.shape
    vocab = w.shape[0]
    g_nll = None if grad_nll is None else grad_nll.detach().to(device=dev, dtype=torch.float32).contiguous()
    g_ent = None if grad_entropy is None else grad_entropy.detach().to(device=dev, dtype=torch.float32).contiguous()
    grad_x = torch.empty((n_rows, h8), dtype=dtype, device=dev) if need_x else None
    grad_w = torch.empty((vocab, h8), dtype=dtype, device=dev) if need_w else None
    if (need_x or need_w) and not (g_nll is None and g_ent is None):
        prob = _fused_problem(x, w, target, temperature, ignore_index)
        with _fl._device_guard(dev):
            ws = _workspace(lib.flce_b200_sce_workspace_bytes(C.byref(prob), _lib.PHASE_BACKWARD, SLAB_BUDGET_BYTES), dev)
            check(lib.flce_b200_sce_backward(C.byref(prob), _ptr(lse), _ptr(entropy), _ptr(g_nll), _ptr(g_ent), _DTYPES[dtype],
                                             _ptr(grad_x), _ptr(grad_w), _ptr(ws), ws.numel(), SLAB_BUDGET_BYTES, _fl._stream(dev)))
    else:
        for g in (grad_x, grad_w):
            if g is not None:
                g.zero_()
    if h8 != hidden:
        grad_x = None if grad_x is None else grad_x[:, :hidden].contiguous()
        grad_w = None if grad_w is None else grad_w[:, :hidden].contiguous()
    return grad_x, grad_w, None, None, None, None


class _ScaledCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden_states, vocab_weights, input_ids, temperature, ignore_index, return_entropy):
        ctx.set_materialize_grads(False)
        _validate_inputs(hidden_states, vocab_weights, input_ids)
        _validate_temperature(temperature)
        _fl._require_cuda(hidden_states)
        # backward recomputes the logits from the operands: remember their versions so that an in-place change in
        # between is reported (what ctx.save_for_backward would do) instead of mixing new logits with the old lse
        ctx.sce_operands = ((hidden_states, hidden_states._version), (vocab_weights, vocab_weights._version))
        if MODE == "fused" and hidden_states.dtype in (torch.bfloat16, torch.float16):
            return _fused_forward(ctx, hidden_states, vocab_weights, input_ids, temperature, ignore_index, return_entropy)
        dev, dtype = hidden_states.device, hidden_states.dtype
        lib = ck._lib_handle()
        need_grads = any(ctx.needs_input_grad[:2])
        head = ck.Head(hidden_states, vocab_weights, need_grads=need_grads)
        target = input_ids.detach().contiguous()
        n_rows, vocab = head.n_rows, head.vocab
        chunk_rows, n_chunks = ck.plan_chunks(n_rows, head.slab_bytes_per_row())
        slab = head.new_slab(chunk_rows)
        nll = torch.empty(n_rows, dtype=torch.float32, device=dev)
        entropy = torch.empty(n_rows, dtype=torch.float32, device=dev)
        lse = torch.empty(n_rows, dtype=torch.float32, device=dev)
        with _fl._device_guard(dev):
            for c in range(n_chunks):
                r0 = c * chunk_rows
                rows = min(chunk_rows, n_rows - r0)
                head.logits(r0, rows, slab)
                check(lib.flce_b200_scaled_ce_rows(
                    _ptr(slab), slab.stride(0), _DTYPES[dtype], rows, vocab, _ptr(target[r0:r0 + rows]), int(ignore_index),
                    float(temperature), _ptr(nll[r0:r0 + rows]), _ptr(entropy[r0:r0 + rows]), _ptr(lse[r0:r0 + rows]),
                    _fl._stream(dev)))
        ctx.sce = (head, target, lse, entropy, float(temperature), int(ignore_index), chunk_rows)
        if return_entropy:
            return nll, entropy.to(dtype)
        return nll

    @staticmethod
    def backward(ctx, grad_nll, grad_entropy=None):
        for tensor, version in ctx.sce_operands:
            if tensor._version != version:
                raise RuntimeError("one of the variables needed for gradient computation has been modified by an inplace "
                                   f"operation: a {tuple(tensor.shape)} operand of the fused linear scaled cross-entropy is at "
                                   f"version {tensor._version}, expected version {version}")
        if ctx.sce[0] == "fused":
            return _fused_backward(ctx, grad_nll, grad_entropy)
        head, target, lse, entropy, temperature, ignore_index, chunk_rows = ctx.sce
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dev, dtype = head.device, head.dtype
        lib = ck._lib_handle()
        n_rows, vocab = head.n_rows, head.vocab
        n_chunks = (n_rows + chunk_rows - 1) // chunk_rows
        g_nll = None if grad_nll is None else grad_nll.detach().to(device=dev, dtype=torch.float32).contiguous()
        g_ent = None if grad_entropy is None else grad_entropy.detach().to(device=dev, dtype=torch.float32).contiguous()
        grad_x = head.new_grad_input() if need_x else None
        grad_w32 = head.new_grad_weight() if need_w else None
        if (need_x or need_w) and not (g_nll is None and g_ent is None):
            slab = head.new_slab(chunk_rows)      # the forward's slab was released with it
            with _fl._device_guard(dev):
                for c in range(n_chunks):
                    r0 = c * chunk_rows
                    rows = min(chunk_rows, n_rows - r0)
                    head.logits(r0, rows, slab)
                    check(lib.flce_b200_scaled_ce_grad(
                        _ptr(slab), slab.stride(0), _DTYPES[dtype], rows, vocab, _ptr(target[r0:r0 + rows]), ignore_index,
                        temperature, _ptr(lse[r0:r0 + rows]), _ptr(entropy[r0:r0 + rows]),
                        None if g_nll is None else _ptr(g_nll[r0:r0 + rows]),
                        None if g_ent is None else _ptr(g_ent[r0:r0 + rows]), _fl._stream(dev)))
                    head.project(slab, r0, rows, None if grad_x is None else grad_x[r0:r0 + rows], grad_w32)
        elif grad_x is not None:
            grad_x.zero_()
        return head.finish_grad_input(grad_x), head.finish_grad_weight(grad_w32), None, None, None, None


class LigerFusedLinearScaledCrossEntropyFunction:
    """Same entry point as the reference's dispatcher class (``ops/fused_linear_scaled_cross_entropy.py:163-199``):
    ``apply(input, weight, target, temperature, ignore_index, m_tiles_per_cluster, return_entropy)`` returns ``nll`` (fp32,
    ``[M]``) or ``(nll, entropy)`` with the entropy in the operands' dtype; ignored tokens read 0 in both."""

    @staticmethod
    def apply(_input, weight, target, temperature=1.0, ignore_index=-100, m_tiles_per_cluster=1, return_entropy=False):
        if not isinstance(m_tiles_per_cluster, int) or isinstance(m_tiles_per_cluster, bool):
            raise TypeError("m_tiles_per_cluster must be an int")
        if m_tiles_per_cluster < 1:
            raise ValueError("m_tiles_per_cluster must be >= 1")
        if not isinstance(return_entropy, bool):
            raise TypeError("return_entropy must be a bool")
        return _ScaledCrossEntropy.apply(_input, weight, target, temperature, ignore_index, return_entropy)


__all__ = ["LigerFusedLinearScaledCrossEntropyFunction"]
