"""Shared host plumbing of the chunked head losses (fused linear JSD, fused linear scaled cross-entropy).

Both run the reference's loop over token chunks (``src/liger_kernel/ops/fused_linear_jsd.py:44-140``,
``src/liger_kernel/ops/fused_linear_scaled_cross_entropy.py:113-160``): logits of a chunk into a bounded slab, a row
kernel over the slab, two projections out of it.  Here every matrix product is the library's tcgen05 GEMM
(``flce_b200_gemm_accumulate``) and every row pass one of its SIMT kernels; torch only holds the memory.

16-bit operands: the slab has the operands' dtype (the reference rounds its chunk logits to that dtype too) and the
row kernel leaves the logit gradient in it, ready to be a GEMM operand.  fp32 operands: the tensor cores take 16-bit
inputs, so x and w are split into bf16 terms on the device (``flce_b200_split_fp32``): six term products give the fp32
logits (x.w to about 2^-24), the slab is fp32, and the logit gradient is split into two bf16 terms for the projections
(three accumulating GEMMs each: dz0.w0 + dz0.w1 + dz1.w0, about 2^-17 per product).
"""

from __future__ import annotations

import ctypes as C

import torch

from .. import _lib
from .._lib import check
from . import fused_linear_cross_entropy as _fl
from .fused_linear_cross_entropy import _DTYPES, _pad_hidden, _ptr

# bytes of slab memory a chunk may use (logits of one head for the scaled cross-entropy, of both for JSD, plus the
# 16-bit copy of the logit gradient when the operands are fp32)
SLAB_BUDGET_BYTES = 1 << 30


def _lib_handle():
    return _fl.lib      # one handle for the whole package (tests swap it there)


def slab_pitch(vocab: int) -> int:
    """Row pitch of a logits slab in elements: a multiple of 64 keeps every row 16-byte aligned for all dtypes."""
    return (vocab + 63) // 64 * 64


def plan_chunks(n_rows: int, bytes_per_row: int, budget: int = 0):
    """Rows per chunk (a multiple of 256 unless one chunk covers everything) and the number of chunks."""
    budget = budget or SLAB_BUDGET_BYTES
    rows = max(256, budget // bytes_per_row // 256 * 256)
    if rows >= n_rows:
        return n_rows, 1
    n_chunks = (n_rows + rows - 1) // rows
    rows = ((n_rows + n_chunks - 1) // n_chunks + 255) // 256 * 256      # even out the tail
    return rows, (n_rows + rows - 1) // rows


def gemm(a, b, *, m, n, k, ld_a, ld_b, a_mn_major, b_mn_major, out=None, ld_out=0, acc=None, ld_acc=0):
    """v = A . B^T (+ acc); A is [m, k] (k contiguous) or, MN-major, [k, m]; B is [n, k] or [k, n]; see
    ``flce_b200_gemm_accumulate``.  ``a`` / ``b`` / ``out`` / ``acc`` are tensors whose storage starts at the matrix."""
    out_dtype = _DTYPES[out.dtype] if out is not None else _DTYPES[a.dtype]
    check(_lib_handle().flce_b200_gemm_accumulate(
        _ptr(a), _ptr(b), _ptr(acc), _ptr(out), m, n, k, ld_a, ld_b, ld_acc, ld_out, _DTYPES[a.dtype], out_dtype,
        int(a_mn_major), int(b_mn_major), 1, _fl._stream(a.device)))


class Head:
    """One language-model head ``x [N, H] -> logits [N, V]`` prepared for the chunk loop: operand copies the TMA engine
    can read (hidden size zero-padded to a multiple of 8; bf16 term splits for fp32), and the three products."""

    def __init__(self, x: torch.Tensor, w: torch.Tensor, need_grads: bool):
        if x.dtype not in _DTYPES:
            raise TypeError(f"unsupported dtype {x.dtype}")
        self.device, self.dtype = x.device, x.dtype
        self.n_rows, self.hidden = x.shape
        self.vocab = w.shape[0]
        self.pitch = slab_pitch(self.vocab)
        self.fp32 = x.dtype == torch.float32
        self.h8 = (self.hidden + 7) // 8 * 8
        x, w = x.detach(), w.detach()
        if self.fp32:
            self.x_fwd = _fl._split_fp32(x, _fl._X_TERMS, self.h8)          # [N, 6 h8]
            self.w_fwd = _fl._split_fp32(w, _fl._W_TERMS, self.h8)          # [V, 6 h8]
            self.x2 = _fl._split_fp32(x, _fl._PROJ_TERMS, self.h8) if need_grads else None    # [N, 2 h8]: x0 | x1
            self.w2 = _fl._split_fp32(w, _fl._PROJ_TERMS, self.h8) if need_grads else None    # [V, 2 h8]: w0 | w1
            self.grad_dtype = torch.float32
        else:
            self.x_fwd = _pad_hidden(x)
            self.w_fwd = _pad_hidden(w)
            self.grad_dtype = self.dtype
        self.dz2 = None

    # bytes of slab memory one token row needs (logits slab + the split gradient for fp32)
    def slab_bytes_per_row(self) -> int:
        return self.pitch * (4 + 4 if self.fp32 else self.x_fwd.element_size())

    def new_slab(self, rows: int) -> torch.Tensor:
        return torch.empty((rows, self.pitch), dtype=self.dtype, device=self.device)

    def logits(self, r0: int, rows: int, slab: torch.Tensor):
        """slab[:rows, :V] = x[r0:r0+rows] . w^T"""
        xc = self.x_fwd[r0:r0 + rows]
        gemm(xc, self.w_fwd, m=rows, n=self.vocab, k=xc.shape[1], ld_a=xc.stride(0), ld_b=self.w_fwd.stride(0),
             a_mn_major=False, b_mn_major=False, out=slab, ld_out=slab.stride(0))

    def _split_gradient(self, slab: torch.Tensor, rows: int):
        """fp32 logit gradient -> [dz0 | dz1] bf16 column blocks of `pitch` columns each."""
        if self.dz2 is None or self.dz2.shape[0] < rows:
            self.dz2 = torch.empty((slab.shape[0], 2 * self.pitch), dtype=torch.bfloat16, device=self.device)
        pat = (C.c_int32 * 2)(0, 1)
        lib = _lib_handle()
        for s0 in range(0, rows, 65535):
            n = min(65535, rows - s0)
            check(lib.flce_b200_split_fp32(_ptr(slab[s0:s0 + n]), n, self.vocab, slab.stride(0), _ptr(self.dz2[s0:s0 + n]),
                                           self.dz2.stride(0), self.pitch, pat, 2, _lib.FLCE_BF16, _fl._stream(self.device)))

    def project(self, slab: torch.Tensor, r0: int, rows: int, grad_rows, grad_weight32):
        """With dZ = slab[:rows, :V]: grad_rows[rows, h8] = dZ . w (when not None) and grad_weight32[V, h8] += dZ^T . x[r0:r0+rows]
        (when not None; fp32 accumulator across chunks)."""
        v, h8, p = self.vocab, self.h8, self.pitch
        if not self.fp32:
            xc = self.x_fwd[r0:r0 + rows]
            if grad_rows is not None:
                gemm(slab, self.w_fwd, m=rows, n=h8, k=v, ld_a=slab.stride(0), ld_b=self.w_fwd.stride(0), a_mn_major=False,
                     b_mn_major=True, out=grad_rows, ld_out=grad_rows.stride(0))
            if grad_weight32 is not None:
                gemm(slab, xc, m=v, n=h8, k=rows, ld_a=slab.stride(0), ld_b=xc.stride(0), a_mn_major=True, b_mn_major=True,
                     acc=grad_weight32, ld_acc=grad_weight32.stride(0))
            return
        self._split_gradient(slab, rows)
        dz0, dz1 = self.dz2, self.dz2[:, p:]                  # views: same pitch 2p, second block starts p columns in
        ld_dz = self.dz2.stride(0)
        if grad_rows is not None:
            w0, w1 = self.w2, self.w2[:, h8:]
            ld_w = self.w2.stride(0)
            terms = ((dz0, w0), (dz0, w1), (dz1, w0))
            for i, (a, b) in enumerate(terms):
                gemm(a, b, m=rows, n=h8, k=v, ld_a=ld_dz, ld_b=ld_w, a_mn_major=False, b_mn_major=True,
                     out=grad_rows if i == 0 else None, ld_out=grad_rows.stride(0) if i == 0 else 0,
                     acc=None if i == 0 else grad_rows, ld_acc=0 if i == 0 else grad_rows.stride(0))
        if grad_weight32 is not None:
            x2 = self.x2[r0:r0 + rows]
            x0, x1 = x2, x2[:, h8:]
            ld_x = x2.stride(0)
            for a, b in ((dz0, x0), (dz0, x1), (dz1, x0)):
                gemm(a, b, m=v, n=h8, k=rows, ld_a=ld_dz, ld_b=ld_x, a_mn_major=True, b_mn_major=True, acc=grad_weight32,
                     ld_acc=grad_weight32.stride(0))

    def new_grad_input(self):
        return torch.empty((self.n_rows, self.h8), dtype=self.grad_dtype, device=self.device)

    def new_grad_weight(self):
        return torch.zeros((self.vocab, self.h8), dtype=torch.float32, device=self.device)

    def finish_grad_input(self, g):
        return g if g is None or self.h8 == self.hidden else g[:, :self.hidden].contiguous()

    def finish_grad_weight(self, g32):
        if g32 is None:
            return None
        g = g32 if self.h8 == self.hidden else g32[:, :self.hidden]
        return g.to(self.dtype) if self.dtype != torch.float32 else g.contiguous()
