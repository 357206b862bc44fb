"""Fused linear cross-entropy on B200: host side of the operator.

Same call surface as the reference's ``src/liger_kernel/ops/fused_linear_cross_entropy.py``
(``fused_linear_cross_entropy_forward`` / ``..._backward`` /
``LigerFusedLinearCrossEntropyFunction``), but every number is produced by
``libflce_b200.so`` (tcgen05 + TMA kernels) through its C ABI.  torch is used for device
memory and the current stream only.  There is no CPU or eager fallback.

Two execution modes (``MODE`` below, or the environment variable ``LIGER_B200_FLCE_MODE``):
* ``"recompute"``: forward computes only the loss (sweep 1); ``backward`` recomputes the logits tile by tile
  (sweep 2) with the upstream gradient folded in.  8.N.H.V tensor FLOPs, smallest memory, any reduction.
* ``"single_sweep"``: when a gradient is required, the reduction is mean or sum and the operands are 16-bit, forward
  also forms the gradients, as the reference does (``ops/fused_linear_cross_entropy.py:395-435``), from a bounded 16-bit
  copy of each token chunk's logits: 6.N.H.V tensor FLOPs.  The first ``backward`` hands the stored gradients off
  (scaled on the device if the upstream gradient is not 1); a repeated ``backward`` falls back to the recompute sweep.
* ``"auto"`` (default): ``single_sweep`` wherever it applies, ``recompute`` elsewhere (``reduction="none"``, fp32
  operands, forward-only calls).

Differences from the reference that a caller can observe:
* logits stay fp32 from accumulator to loss (the reference rounds them to the input dtype).
* there is no host synchronisation (the reference reads the non-ignored count with ``.item()``).
"""

from __future__ import annotations

import ctypes as C
import os
import threading
from typing import Optional

import torch

from .. import _lib
from .._lib import BackwardArgs, ForwardOut, FusedArgs, Problem, check, lib

_DTYPES = {torch.bfloat16: _lib.FLCE_BF16, torch.float16: _lib.FLCE_FP16, torch.float32: _lib.FLCE_FP32}
_REDUCTIONS = {"mean": _lib.FLCE_MEAN, "sum": _lib.FLCE_SUM, "none": _lib.FLCE_NONE}

# bytes of logit-gradient slab the backward sweep may use (N x slab columns, 16-bit)
SLAB_BUDGET_BYTES = 1 << 30
# bytes of logits copy the single-sweep mode may use (chunk rows x V, 16-bit)
CHUNK_BUDGET_BYTES = 5 << 29
MODE = os.environ.get("LIGER_B200_FLCE_MODE", "auto")
# What the single-sweep mode keeps of a chunk's logits: "auto" (their exponentials wherever that form applies, else the
# logits), "logits" or "exp" (see flce_store_mode_t in include/flce_b200.h).
STORE_MODE = os.environ.get("LIGER_B200_FLCE_STORE", "auto")
_STORE_MODES = {"auto": _lib.STORE_AUTO, "logits": _lib.STORE_LOGITS, "exp": _lib.STORE_EXP}
# Read back the count of out-of-range targets after forward and raise, as the reference's stand-alone cross-entropy and
# its sm_100 FLCE do (``ops/cross_entropy.py:389-392``).  Costs a host synchronisation, so it is off by default.
CHECK_TARGETS = os.environ.get("LIGER_B200_CHECK_TARGETS", "0") == "1"
# Move rows whose target is ignore_index to the end (on the device, no host sync) and let the sweeps skip the token
# tiles that hold none of the others: the tensor work shrinks by the ignored fraction.  16-bit inputs, both modes.
SKIP_IGNORED = os.environ.get("LIGER_B200_FLCE_SKIP_IGNORED", "1") == "1"


def _raise_on_bad_targets(norm, vocab):
    bad = int(norm[3].item())
    assert bad == 0, f"Target out of bounds: {bad} targets are neither ignore_index nor in [0, {vocab})"


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _device_guard(device):
    """Make `device` current for the calls inside (the library works on the current device)."""
    return torch.cuda.device(device)


def _require_cuda(t: torch.Tensor):
    if t.device.type != "cuda":
        raise RuntimeError("liger_kernel_b200 runs on CUDA (sm_100a) tensors only; there is no CPU path")


def _pad_hidden(t: torch.Tensor, mult: int = 8) -> torch.Tensor:
    """Rows must be 16-byte multiples for the TMA engine; zero-pad the hidden dimension if needed."""
    h = t.shape[1]
    if h % mult == 0 and t.is_contiguous():
        return t
    hp = (h + mult - 1) // mult * mult
    if hp == h:
        return t.contiguous()
    out = t.new_zeros((t.shape[0], hp))
    out[:, :h] = t
    return out


_X_TERMS = (0, 0, 0, 1, 1, 2)   # paired with _W_TERMS: x0w0 + x0w1 + x0w2 + x1w0 + x1w1 + x2w0 = x.w to ~2^-24
_W_TERMS = (0, 1, 2, 0, 1, 0)
_PROJ_TERMS = (0, 1)            # projections use the two leading terms: each product good to about 2^-16, so a
                                # gradient element is good to a few 1e-4 of the largest entry at V = 128k, not to fp32 ulp


def _split_fp32(t: torch.Tensor, pattern, block_cols: int) -> torch.Tensor:
    """[rows, cols] fp32 -> [rows, len(pattern) * block_cols] bf16 term blocks (see flce_b200_split_fp32)."""
    t = t.contiguous()
    rows, cols = t.shape
    out = torch.empty((rows, len(pattern) * block_cols), dtype=torch.bfloat16, device=t.device)
    pat = (C.c_int32 * len(pattern))(*pattern)
    with _device_guard(t.device):
        for r0 in range(0, rows, 65535):
            n = min(65535, rows - r0)
            check(lib.flce_b200_split_fp32(_ptr(t[r0:r0 + n]), n, cols, t.stride(0), _ptr(out[r0:r0 + n]), out.stride(0),
                                           block_cols, pat, len(pattern), _lib.FLCE_BF16, _stream(t.device)))
    return out


class _Prepared:
    """Validated, device-resident operands of one FLCE call and the matching C struct."""

    def __init__(self, _input, weight, target, bias, ce_weight, ignore_index, lse_square_scale, label_smoothing,
                 reduction, softcap, use_token_scaling, vocab_total=None, vocab_offset=0, want_argmax=True,
                 allow_compact=False, rms_norm=None):
        # rms_norm: dict(weight, eps, offset, casting_mode) when ``_input`` holds the hidden states *before* the decoder's
        # final RMSNorm; the norm is then applied by the gather that moves the rows that matter to the front
        _require_cuda(_input)
        if _input.dim() != 2 or weight.dim() != 2 or _input.shape[1] != weight.shape[1]:
            raise ValueError(f"expected _input [BT, H] and weight [V, H], got {tuple(_input.shape)} and {tuple(weight.shape)}")
        if target.dim() != 1 or target.shape[0] != _input.shape[0]:
            raise ValueError(f"target must be [BT]={_input.shape[0]}, got {tuple(target.shape)}")
        if _input.dtype != weight.dtype:
            raise TypeError(f"_input ({_input.dtype}) and weight ({weight.dtype}) must share a dtype")
        if _input.dtype not in _DTYPES:
            raise TypeError(f"unsupported dtype {_input.dtype}")
        if reduction not in _REDUCTIONS:
            raise ValueError(f"reduction must be 'mean', 'sum' or 'none'. Got: {reduction}")
        if bias is not None and bias.shape != (weight.shape[0],):
            raise ValueError(f"bias must be [V]={weight.shape[0]}, got {tuple(bias.shape)}")
        if ce_weight is not None:
            assert ce_weight.shape[0] == weight.shape[0], f"If given, weight has to be a Tensor of size V. Got: {ce_weight.shape}"
            assert torch.is_floating_point(ce_weight), f"If given, weight has to be a Tensor of floating point dtype. Got: {ce_weight.dtype}"
        self.device = _input.device
        self.n_rows, self.hidden = _input.shape
        self.vocab = weight.shape[0]
        self.dtype = _input.dtype
        self.reduction = reduction
        self.split = self.dtype == torch.float32
        if self.split:
            # fp32 inputs: 16-bit term splits side by side, so the same bf16 tensor-core kernels give fp32-level logits
            self.block = (self.hidden + 7) // 8 * 8
            x32, w32 = _input.detach(), weight.detach()
            self.x = _split_fp32(x32, _X_TERMS, self.block)
            self.w = _split_fp32(w32, _W_TERMS, self.block)
            self.proj_x = _split_fp32(x32, _PROJ_TERMS, self.block)
            self.proj_w = _split_fp32(w32, _PROJ_TERMS, self.block)
        else:
            self.x = _pad_hidden(_input.detach())
            self.w = _pad_hidden(weight.detach())
        self.target = target.detach().to(device=self.device, dtype=torch.int64).contiguous()
        self.bias = None if bias is None else bias.detach().to(device=self.device, dtype=torch.float32).contiguous()
        self.ce_weight = None if ce_weight is None else ce_weight.detach().to(device=self.device, dtype=torch.float32).contiguous()
        p = Problem()
        p.n_rows, p.hidden, p.vocab = self.n_rows, self.x.shape[1], self.vocab
        p.vocab_total = self.vocab if vocab_total is None else int(vocab_total)
        p.vocab_offset = int(vocab_offset)
        p.ld_x, p.ld_w = self.x.stride(0), self.w.stride(0)
        p.dtype = _lib.FLCE_BF16 if self.split else _DTYPES[self.dtype]
        p.reduction = _REDUCTIONS[reduction]
        p.ignore_index = int(ignore_index)
        p.label_smoothing = float(label_smoothing)
        p.lse_square_scale = float(lse_square_scale)
        p.softcap = 0.0 if softcap is None else float(softcap)
        p.use_token_scaling = int(bool(use_token_scaling))
        p.flags = _lib.FLAG_ARGMAX if want_argmax else 0
        p.x, p.w, p.target = self.x.data_ptr(), self.w.data_ptr(), self.target.data_ptr()
        p.bias = None if self.bias is None else self.bias.data_ptr()
        p.ce_weight = None if self.ce_weight is None else self.ce_weight.data_ptr()
        self.problem = p
        self.compacted = False
        self.rms_norm = None
        if rms_norm is not None:
            if self.split or self.hidden % 8 != 0 or self.hidden > 16384:
                raise NotImplementedError("the fused RMSNorm needs bf16 / fp16 hidden states with a hidden size that is a "
                                          "multiple of 8 and at most 16384")
            mode = {"llama": 0, "gemma": 1}.get(rms_norm["casting_mode"])
            if mode is None:
                raise NotImplementedError(f"casting_mode must be 'llama' or 'gemma', got {rms_norm['casting_mode']!r}")
            gamma = rms_norm["weight"].detach().to(device=self.device, dtype=self.dtype).contiguous()
            if gamma.shape != (self.hidden,):
                raise ValueError(f"the norm weight must be [H]={self.hidden}, got {tuple(gamma.shape)}")
            self.rms_norm = dict(weight=gamma, eps=float(rms_norm["eps"]), offset=float(rms_norm["offset"]), mode=mode)
            self.raw_hidden = self.x
            self._compact()
        elif allow_compact and SKIP_IGNORED and not self.split:
            self._compact()

    def _compact(self):
        """Stable-partition the rows (targets that are not ignore_index first) and point the problem at the result."""
        n, dev = self.n_rows, self.device
        xc = torch.empty((n, self.x.shape[1]), dtype=self.x.dtype, device=dev)
        tc = torch.empty_like(self.target)
        self.perm = torch.empty(n, dtype=torch.int32, device=dev)
        self.active = torch.empty(1, dtype=torch.int32, device=dev)
        with _device_guard(dev):
            if self.rms_norm is not None:
                rn = self.rms_norm
                self.rstd = torch.empty(n, dtype=torch.float32, device=dev)
                check(lib.flce_b200_compact_rows_rmsnorm(C.byref(self.problem), _ptr(rn["weight"]), rn["eps"], rn["offset"],
                                                         rn["mode"], _ptr(xc), _ptr(tc), _ptr(self.perm), _ptr(self.active),
                                                         _ptr(self.rstd), _stream(dev)))
            else:
                check(lib.flce_b200_compact_rows(C.byref(self.problem), _ptr(xc), _ptr(tc), _ptr(self.perm), _ptr(self.active),
                                                 _stream(dev)))
        self.x, self.target = xc, tc
        p = self.problem
        p.x, p.ld_x, p.target = xc.data_ptr(), xc.stride(0), tc.data_ptr()
        p.active_rows = self.active.data_ptr()
        self.compacted = True

    def to_token_order(self, t: torch.Tensor, fill=0) -> torch.Tensor:
        """Per-row values in compact order -> token order (rows of ignored tokens are already what they should be)."""
        if not self.compacted:
            return t
        out = torch.full_like(t, fill)
        out[self.perm.long()] = t
        return out

    def to_compact_order(self, t: torch.Tensor) -> torch.Tensor:
        return t[self.perm.long()] if self.compacted else t

    def rows_to_token_order(self, m: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """A compact [n_rows, cols] matrix (grad_input) -> token order, zeros on ignored rows."""
        if m is None or not self.compacted:
            return m
        out = torch.empty_like(m)
        with _device_guard(self.device):
            check(lib.flce_b200_scatter_rows(_ptr(m), m.shape[1] * m.element_size(), _ptr(self.perm), _ptr(self.active),
                                             m.shape[0], _ptr(out), _stream(self.device)))
        return out

    def rmsnorm_backward(self, grad_normed: torch.Tensor):
        """Gradient with respect to the normalised rows (compact order) -> (grad_hidden in token order, zeros on ignored rows;
        grad of the norm weight, fp32)."""
        rn, dev = self.rms_norm, self.device
        raw = self.raw_hidden
        grad_hidden = torch.empty_like(raw)
        grad_gamma = torch.empty(self.hidden, dtype=torch.float32, device=dev)
        partials = torch.empty(lib.flce_b200_rmsnorm_partial_floats(self.hidden), dtype=torch.float32, device=dev)
        with _device_guard(dev):
            check(lib.flce_b200_rmsnorm_scatter_backward(
                _ptr(grad_normed), grad_normed.stride(0), _ptr(raw), raw.stride(0), _DTYPES[self.dtype], self.n_rows, self.hidden,
                _ptr(rn["weight"]), _ptr(self.rstd), _ptr(self.perm), _ptr(self.active), rn["offset"], rn["mode"],
                _ptr(grad_hidden), grad_hidden.stride(0), _ptr(grad_gamma), _ptr(partials), _stream(dev)))
        return grad_hidden, grad_gamma

    def workspace(self, phase: int, budget: int = 0) -> torch.Tensor:
        nbytes = lib.flce_b200_workspace_bytes(C.byref(self.problem), phase, budget)
        if nbytes == 0:
            raise _lib.FlceError(f"libflce_b200: {lib.flce_b200_last_error().decode()}")
        return torch.empty(nbytes, dtype=torch.uint8, device=self.device)


def _forward_outputs(prep: _Prepared):
    n, dev = prep.n_rows, prep.device
    f32 = dict(dtype=torch.float32, device=dev)
    return dict(
        lse=torch.empty(n, **f32), target_prob=torch.empty(n, **f32), loss_rows=torch.empty(n, **f32),
        z_loss_rows=torch.empty(n, **f32), correct_rows=torch.empty(n, **f32),
        predicted_tokens=torch.empty(n, dtype=torch.int64, device=dev), scalars=torch.empty(4, **f32),
    )


def _as_forward_out(o) -> ForwardOut:
    f = ForwardOut()
    for k, v in o.items():
        setattr(f, k, v.data_ptr())
    return f


def flce_forward_device(prep: _Prepared):
    """Run count + sweep 1 + finalize.  Returns (outputs dict, norm[4], rowstats[6, N])."""
    with _device_guard(prep.device):
        norm = torch.empty(4, dtype=torch.float32, device=prep.device)
        rowstats = torch.empty((_lib.ROWSTAT_PLANES, prep.n_rows), dtype=torch.float32, device=prep.device)
        out = _forward_outputs(prep)
        ws = prep.workspace(_lib.PHASE_FORWARD)
        fo = _as_forward_out(out)
        check(lib.flce_b200_forward(C.byref(prep.problem), _ptr(norm), _ptr(rowstats), C.byref(fo), _ptr(ws),
                                    ws.numel(), _stream(prep.device)))
    return out, norm, rowstats


def flce_backward_device(prep: _Prepared, lse, target_prob, norm, grad_output, need_input=True, need_weight=True,
                         need_bias=False, grad_dtype=None, slab_budget=None, slab_hook=None):
    """Run sweep 2.  Returns (grad_input, grad_weight, grad_bias) in the padded hidden size of ``prep``.

    ``slab_hook(first_row, last_row, grad_weight)``, if given, is called after the kernels of each vocabulary slab
    have been enqueued, with the range of ``grad_weight`` rows that slab completes (used to overlap an all-reduce)."""
    dev = prep.device
    gd = prep.dtype if grad_dtype is None else grad_dtype
    budget = SLAB_BUDGET_BYTES if slab_budget is None else int(slab_budget)
    hp = prep.x.shape[1]
    if prep.split:
        gd = torch.float32
        hp = prep.proj_x.shape[1]
    with _device_guard(dev):
        gx = torch.empty((prep.n_rows, hp), dtype=gd, device=dev) if need_input else None
        gw = torch.empty((prep.vocab, hp), dtype=gd, device=dev) if need_weight else None
        gb = torch.empty(prep.vocab, dtype=torch.float32, device=dev) if need_bias else None
        args = BackwardArgs()
        if prep.split:
            args.proj_x, args.proj_x_cols, args.ld_proj_x = prep.proj_x.data_ptr(), hp, prep.proj_x.stride(0)
            args.proj_w, args.proj_w_cols, args.ld_proj_w = prep.proj_w.data_ptr(), hp, prep.proj_w.stride(0)
            args.split_logit_grad, args.lo_cols_x, args.lo_cols_w = 1, prep.block, prep.block
        args.lse, args.target_prob, args.norm = lse.data_ptr(), target_prob.data_ptr(), norm.data_ptr()
        go = None
        if grad_output is not None:
            go = grad_output.detach().to(device=dev, dtype=torch.float32).contiguous().reshape(-1)
            if go.numel() not in (1, prep.n_rows):
                raise ValueError(f"grad_output must have 1 or {prep.n_rows} elements, got {go.numel()}")
            args.grad_output = go.data_ptr()
            args.grad_output_per_row = int(go.numel() == prep.n_rows and prep.reduction == "none")
        args.grad_dtype = _DTYPES[gd]
        args.grad_input = None if gx is None else gx.data_ptr()
        args.grad_weight = None if gw is None else gw.data_ptr()
        args.grad_bias = None if gb is None else gb.data_ptr()
        ws = prep.workspace(_lib.PHASE_BACKWARD_SPLIT if prep.split else _lib.PHASE_BACKWARD, budget)
        if slab_hook is None:
            check(lib.flce_b200_backward(C.byref(prep.problem), C.byref(args), _ptr(ws), ws.numel(), budget, _stream(dev)))
        else:
            n_slabs, slab_cols = C.c_int32(0), C.c_int64(0)
            check(lib.flce_b200_backward_plan(C.byref(prep.problem), budget, C.byref(n_slabs), C.byref(slab_cols)))
            for s in range(n_slabs.value):
                args.slab_begin, args.slab_end = s, s + 1
                check(lib.flce_b200_backward(C.byref(prep.problem), C.byref(args), _ptr(ws), ws.numel(), budget,
                                             _stream(dev)))
                slab_hook(s * slab_cols.value, min(prep.vocab, (s + 1) * slab_cols.value), gw)
        if prep.split:  # sum the term blocks: (dZ_hi + dZ_lo).t0 + dZ_hi.t1
            b = prep.block
            gx = None if gx is None else gx[:, :b] + gx[:, b:2 * b]
            gw = None if gw is None else gw[:, :b] + gw[:, b:2 * b]
    return gx, gw, gb


def flce_single_sweep_device(prep: _Prepared, need_input=True, need_weight=True, need_bias=False, grad_dtype=None,
                             chunk_budget=None, norm_in=None, after_grad_weight=None, reserve_sms=0, shard_hooks=None):
    """Loss and gradients (for an upstream gradient of 1) in one pass over token chunks.
    Returns (outputs dict, norm, grad_input, grad_weight, grad_bias) in the padded hidden size of ``prep``.
    ``norm_in``: normalisers counted elsewhere (a token-sharded caller passes the all-reduced ones).
    ``after_grad_weight(grad_weight)``: called on this thread once the launch that completes grad_weight is enqueued,
    before the last grad_input GEMM, which then leaves ``reserve_sms`` SMs free (room for the caller's collective).
    ``shard_hooks``: for a vocabulary shard, a dict of the three exchanges (``flce_fused_args_t`` in include/flce_b200.h),
    here with tensors instead of pointers: ``exchange_shift(shift[n_rows])``, ``exchange_rowstats(stats[6, rows], first_row)``
    (both update their argument in place) and ``after_grad_input(grad_input[first_row:first_row+rows], first_row)``."""
    dev = prep.device
    gd = prep.dtype if grad_dtype is None else grad_dtype
    budget = CHUNK_BUDGET_BYTES if chunk_budget is None else int(chunk_budget)
    hp = prep.x.shape[1]
    with _device_guard(dev):
        norm = torch.empty(4, dtype=torch.float32, device=dev)
        out = _forward_outputs(prep)
        fo = _as_forward_out(out)
        gx = torch.empty((prep.n_rows, hp), dtype=gd, device=dev) if need_input else None
        gw = torch.empty((prep.vocab, hp), dtype=gd, device=dev) if need_weight else None
        gb = torch.empty(prep.vocab, dtype=torch.float32, device=dev) if need_bias else None
        args = FusedArgs()
        args.out = C.pointer(fo)
        args.norm = norm.data_ptr()
        args.grad_dtype = _DTYPES[gd]
        args.grad_input = None if gx is None else gx.data_ptr()
        args.grad_weight = None if gw is None else gw.data_ptr()
        args.grad_bias = None if gb is None else gb.data_ptr()
        args.store_mode = _STORE_MODES[STORE_MODE]
        if norm_in is not None:
            norm.copy_(norm_in)
            args.norm_given = 1
        hook = None
        if after_grad_weight is not None and gw is not None:
            hook = _lib.AFTER_GRAD_WEIGHT_FN(lambda _user: after_grad_weight(gw))     # kept alive until the call returns
            args.after_grad_weight = C.cast(hook, C.c_void_p)
            args.reserve_sms = int(reserve_sms)
        ws = prep.workspace(_lib.PHASE_FUSED, budget)
        keep = []
        if shard_hooks is not None:
            def view(ptr, count):          # `count` floats at a pointer the library hands out, as a tensor (no copy)
                return _float_tensor_at(ptr, count, dev)

            def on_shift(_user, ptr, n):
                shard_hooks["exchange_shift"](view(ptr, n))

            def on_rowstats(_user, ptr, rows, first_row):
                shard_hooks["exchange_rowstats"](view(ptr, _lib.ROWSTAT_PLANES * rows).view(_lib.ROWSTAT_PLANES, rows), first_row)

            def on_grad_input(_user, _ptr_unused, rows, first_row):
                shard_hooks["after_grad_input"](gx[first_row:first_row + rows], first_row)

            keep = [_lib.EXCHANGE_SHIFT_FN(on_shift), _lib.EXCHANGE_ROWSTATS_FN(on_rowstats), _lib.AFTER_GRAD_INPUT_FN(on_grad_input)]
            args.exchange_shift, args.exchange_rowstats, args.after_grad_input = (C.cast(f, C.c_void_p) for f in keep)
            args.reserve_sms = int(reserve_sms)
        check(lib.flce_b200_forward_backward(C.byref(prep.problem), C.byref(args), _ptr(ws), ws.numel(), budget, _stream(dev)))
        del hook, keep
    return out, norm, gx, gw, gb


def scale_gradient_(t: Optional[torch.Tensor], scale: torch.Tensor):
    """In-place ``t *= scale`` with a device-resident fp32 scalar; a no-op on the device when the scalar is 1."""
    if t is None:
        return None
    with _device_guard(t.device):
        check(lib.flce_b200_scale_gradient(_ptr(t), t.numel(), _DTYPES[t.dtype], _ptr(scale), _stream(t.device)))
    return t


class _CudaFloats:
    """fp32 device memory at a raw pointer, in the form torch.as_tensor understands (CUDA array interface)."""

    def __init__(self, ptr, count):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def _float_tensor_at(ptr: int, count: int, device) -> torch.Tensor:
    if device.type == "cuda":
        return torch.as_tensor(_CudaFloats(ptr, count), device=device)
    return torch.frombuffer((C.c_char * (count * 4)).from_address(ptr), dtype=torch.float32, count=count)


def _autocast_operands(_input, weight, bias):
    if torch.is_autocast_enabled("cuda"):
        dt = torch.get_autocast_dtype("cuda")
        _input = _input.to(dt)
        weight = weight.to(dt)
        bias = None if bias is None else bias.to(dt)
    return _input, weight, bias


def fused_linear_cross_entropy_forward(
    _input, weight, target, ce_weight=None, bias=None, ignore_index=-100, lse_square_scale=0.0, label_smoothing=0.0,
    reduction="mean", softcap=None, return_z_loss=False, accum_dtype=None, use_token_scaling=False,
    return_token_accuracy=False, return_predicted_tokens=False,
):
    """Loss side of the operator (``ops/fused_linear_cross_entropy.py:21-289`` of the reference).

    Returns ``(loss, z_loss, token_accuracy, predicted_tokens, saved)`` where ``saved`` carries what
    ``fused_linear_cross_entropy_backward`` needs.  ``accum_dtype`` is accepted for signature
    compatibility: weight gradients here are reduced over all tokens in fp32 tensor memory and written
    once, so there is no lower-precision accumulation to opt out of.
    """
    assert isinstance(return_z_loss, bool), f"return_z_loss must be True or False. Got: {return_z_loss}"
    assert isinstance(return_token_accuracy, bool), f"return_token_accuracy must be True or False. Got: {return_token_accuracy}"
    assert isinstance(return_predicted_tokens, bool), f"return_predicted_tokens must be True or False. Got: {return_predicted_tokens}"
    prep = _Prepared(_input, weight, target, bias, ce_weight, ignore_index, lse_square_scale, label_smoothing, reduction,
                     softcap, use_token_scaling, want_argmax=return_token_accuracy or return_predicted_tokens,
                     allow_compact=True)
    out, norm, _rowstats = flce_forward_device(prep)
    out = _results_to_token_order(prep, out)   # lse / target_prob stay in compact order: backward works there
    if CHECK_TARGETS:
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
    saved = (prep, out["lse"], out["target_prob"], norm)
    return loss, z_loss, token_accuracy, predicted_tokens, saved


def fused_linear_cross_entropy_backward(grad_output, saved, need_input=True, need_weight=True, need_bias=False):
    """Gradient side (``ops/fused_linear_cross_entropy.py:205-265,292-336`` of the reference): the upstream
    gradient (scalar, or per token for ``reduction="none"``) is folded into the logit gradient before the
    two projections, so no separate scaling pass exists."""
    prep, lse, target_prob, norm = saved
    if prep.compacted and grad_output is not None and grad_output.numel() == prep.n_rows and prep.reduction == "none":
        grad_output = prep.to_compact_order(grad_output.reshape(-1))
    gx, gw, gb = flce_backward_device(prep, lse, target_prob, norm, grad_output, need_input, need_weight, need_bias)
    gx = prep.rows_to_token_order(gx)
    h = prep.hidden
    if gx is not None and gx.shape[1] != h:
        gx = gx[:, :h].contiguous()
    if gw is not None and gw.shape[1] != h:
        gw = gw[:, :h].contiguous()
    return gx, gw, gb


def _results_to_token_order(prep: _Prepared, out):
    """Per-row results of a compacted call back in token order (lse / target_prob stay compact: backward works there)."""
    if not prep.compacted:
        return out
    return dict(out, loss_rows=prep.to_token_order(out["loss_rows"]), z_loss_rows=prep.to_token_order(out["z_loss_rows"]),
                correct_rows=prep.to_token_order(out["correct_rows"]),
                predicted_tokens=prep.to_token_order(out["predicted_tokens"], fill=-1))


_grad_mode = threading.local()


def _use_single_sweep(reduction, needs, dtype) -> bool:
    return MODE in ("single_sweep", "auto") and reduction in ("mean", "sum") and any(needs) and dtype != torch.float32


class LigerFusedLinearCrossEntropyFunction(torch.autograd.Function):
    """Drop-in for the reference class of the same name (``ops/fused_linear_cross_entropy.py:339-487``):
    same 15 positional arguments, same 4-tuple result, same gradient slots.

    What backward needs is kept with ``ctx.save_for_backward`` (the operands as the caller passed them, the targets, the
    per-row log-sum-exp, target probability and normalisers), as the reference does (``:417,431``): saved-tensor hooks,
    activation offload and torch's check for in-place changes between forward and backward all apply.  The padded,
    compacted or term-split copies the kernels read are rebuilt from those in backward."""

    @classmethod
    def apply(cls, *args, **kwargs):
        # grad mode is always off inside forward(): note here whether the caller is recording, so that an evaluation
        # loop under torch.no_grad() does not pay for gradients nobody will ask for
        _grad_mode.enabled = torch.is_grad_enabled()
        try:
            return super().apply(*args, **kwargs)
        finally:
            _grad_mode.enabled = True

    @staticmethod
    def forward(
        ctx, _input, weight, target, bias=None, ce_weight=None, ignore_index=-100, lse_square_scale=0.0,
        label_smoothing=0.0, reduction="mean", softcap=None, return_z_loss: bool = False, accum_dtype=None,
        use_token_scaling: bool = False, return_token_accuracy: bool = False, return_predicted_tokens: bool = False,
    ):
        assert isinstance(return_z_loss, bool), f"return_z_loss must be True or False. Got: {return_z_loss}"
        assert isinstance(return_token_accuracy, bool), f"return_token_accuracy must be True or False. Got: {return_token_accuracy}"
        assert isinstance(return_predicted_tokens, bool), f"return_predicted_tokens must be True or False. Got: {return_predicted_tokens}"
        ctx.in_dtypes = (_input.dtype, weight.dtype, None if bias is None else bias.dtype)
        x, w, b = _autocast_operands(_input, weight, bias)
        ctx.stored_grads = None
        ctx.has_bias = bias is not None
        ctx.flce_params = dict(ignore_index=ignore_index, lse_square_scale=lse_square_scale, label_smoothing=label_smoothing,
                               reduction=reduction, softcap=softcap, use_token_scaling=use_token_scaling)
        # what autograd will ask for: nothing under torch.no_grad(), whatever the tensors' flags say
        recording = getattr(_grad_mode, "enabled", True)
        needs = (recording and ctx.needs_input_grad[0], recording and ctx.needs_input_grad[1],
                 recording and bias is not None and ctx.needs_input_grad[3])
        want_argmax = return_token_accuracy or return_predicted_tokens
        prep = _Prepared(x, w, target, b, ce_weight, ignore_index, lse_square_scale, label_smoothing, reduction, softcap,
                         use_token_scaling, want_argmax=want_argmax, allow_compact=True)
        if _use_single_sweep(reduction, needs, x.dtype):
            out, norm, gx, gw, gb = flce_single_sweep_device(prep, needs[0], needs[1], needs[2])
            gx = prep.rows_to_token_order(gx)
            ctx.stored_grads = (gx, gw, gb)
        else:
            out, norm, _rowstats = flce_forward_device(prep)
        lse, target_prob = out["lse"], out["target_prob"]
        out = _results_to_token_order(prep, out)
        if CHECK_TARGETS:
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
        ctx.flce_hidden = prep.hidden
        ctx.flce_autocast = (x.dtype, w.dtype)
        ctx.save_for_backward(_input, weight, target, bias, ce_weight, lse, target_prob, norm)
        nondiff = [t for t in (z_loss, token_accuracy, predicted_tokens) if t is not None]
        if nondiff:
            ctx.mark_non_differentiable(*nondiff)
        return loss, z_loss, token_accuracy, predicted_tokens

    @staticmethod
    def backward(ctx, grad_output, grad_output2=None, grad_output3=None, grad_output4=None):
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        need_b = ctx.has_bias and ctx.needs_input_grad[3]
        h = ctx.flce_hidden
        if ctx.stored_grads is not None:
            # single-sweep mode, first backward: hand the stored gradients off (scaled on the device when needed)
            gx, gw, gb = ctx.stored_grads
            ctx.stored_grads = None
            dev = (gx if gx is not None else gw if gw is not None else gb).device
            go = grad_output.detach().to(device=dev, dtype=torch.float32).reshape(1)
            gx = scale_gradient_(gx, go)
            gw = scale_gradient_(gw, go)
            gb = scale_gradient_(gb, go)
            if gx is not None and gx.shape[1] != h:
                gx = gx[:, :h].contiguous()
            if gw is not None and gw.shape[1] != h:
                gw = gw[:, :h].contiguous()
        else:
            _input, weight, target, bias, ce_weight, lse, target_prob, norm = ctx.saved_tensors
            x = _input.to(ctx.flce_autocast[0]) if _input.dtype != ctx.flce_autocast[0] else _input
            w = weight.to(ctx.flce_autocast[1]) if weight.dtype != ctx.flce_autocast[1] else weight
            b = bias if (bias is None or bias.dtype == ctx.flce_autocast[0]) else bias.to(ctx.flce_autocast[0])
            kw = ctx.flce_params
            prep = _Prepared(x, w, target, b, ce_weight, kw["ignore_index"], kw["lse_square_scale"], kw["label_smoothing"],
                             kw["reduction"], kw["softcap"], kw["use_token_scaling"], want_argmax=False, allow_compact=True)
            gx, gw, gb = fused_linear_cross_entropy_backward(grad_output, (prep, lse, target_prob, norm), need_x, need_w, need_b)
        dx, dw, db = ctx.in_dtypes
        gx = None if gx is None else gx.to(dx)
        gw = None if gw is None else gw.to(dw)
        gb = None if gb is None else gb.to(db)
        return (gx, gw, None, gb) + (None,) * 11
