"""The library's SIMT kernels run on the host (tests/emu/): build helper, ctypes binding and a stand-in library
object that sends the entry points made only of SIMT kernels (stand-alone cross-entropy, target counting, row
compaction / scatter, fp32 term split, gradient scaling, the row kernels of the chunked head losses) to the emulation,
so the Python operators can be driven on CPU tensors with real numerics.  The plain tensor-core GEMM entry point is
replaced by torch arithmetic on the same host memory; the fused sweeps stay recording stubs (fake_lib).

Only the tests use this."""

import contextlib
import ctypes as C
import os
import subprocess

import torch

import fake_lib
from fake_lib import _addr

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "emu", "emu_kernels.cpp")
_CSRC = os.path.join(os.path.dirname(_HERE), "liger-kernel_b200", "csrc")
_OUT = os.path.join(_HERE, "emu", "_build", "libflce_emu.so")
_CUDA_INCLUDE = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")

_lib = None


def _stale():
    if not os.path.exists(_OUT):
        return True
    built = os.path.getmtime(_OUT)
    deps = [_SRC, os.path.join(_HERE, "emu", "simt_emulation.hpp")]
    deps += [os.path.join(_CSRC, f) for f in ("row_kernels.cuh", "ce_kernels.cuh", "head_loss_kernels.cuh", "simt_common.cuh", "tile_schedule.cuh", "epilogues.cuh")]
    return any(os.path.getmtime(d) > built for d in deps)


def load():
    """Compile (g++, C++20, host only) when sources changed, then load."""
    global _lib
    if _lib is not None:
        return _lib
    if _stale():
        os.makedirs(os.path.dirname(_OUT), exist_ok=True)
        cmd = ["g++", "-std=c++20", "-O1", "-fPIC", "-shared", "-I", _CUDA_INCLUDE, "-I", _CSRC, "-o", _OUT, _SRC]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError("building the SIMT emulation failed:\n" + done.stderr[-4000:])
    lib = C.CDLL(_OUT)
    P, LL, I, F = C.c_void_p, C.c_longlong, C.c_int, C.c_float
    sigs = {
        "emu_ce_forward": [I, P, LL, LL, LL, P, P, LL, F, F, F, I, P, P, P, P, P, P, P, P, P],
        "emu_ce_backward": [I, P, LL, LL, LL, P, P, LL, F, F, F, I, P, P, P, I, P, LL, P],
        "emu_count": [P, LL, LL, P, LL, LL, F, P],
        "emu_compact_rows": [P, LL, LL, LL, P, LL, P, P, P, P],
        "emu_scatter_rows": [P, LL, P, P, LL, P],
        "emu_compact_rows_rmsnorm": [P, LL, LL, LL, P, LL, I, P, F, F, I, P, P, P, P, P],
        "emu_rmsnorm_scatter_backward": [P, LL, P, LL, I, LL, LL, P, P, P, P, F, I, P, LL, P, P, I],
        "emu_split_fp32": [P, LL, LL, LL, P, LL, LL, P, I, I],
        "emu_dz_inplace": [P, LL, LL, LL, I, P, LL, P, P, P, P, P, F, P, I],
        "emu_reduce_rows": [LL, P, P, P, P, P],
        "emu_colsum": [P, LL, LL, LL, I, P, I, P, I],
        "emu_scale_inplace": [P, LL, I, P],
        "emu_merge_partials": [LL, I, P, P, P, P, P, P],
        "emu_scaled_ce_rows": [P, LL, I, LL, LL, P, LL, F, P, P, P],
        "emu_scaled_ce_grad": [P, LL, I, LL, LL, P, LL, F, P, P, P, P],
        "emu_jsd_rows": [P, LL, P, LL, I, LL, LL, P, LL, F, F, P, F, P],
        "emu_tile_schedule": [I, I, I, I, I, P, P],
        "emu_sce_forward": [P, P, I, I, I, I, LL, LL, P, LL, F, P, P, P, P, P],
        "emu_sce_sweep_dz": [P, P, I, I, I, I, LL, LL, P, LL, F, LL, P, P, P, P, P, LL, I],
        "emu_sweep_stats": [P, P, I, I, I, I, LL, LL, P, P, P, F, LL, P, P, P, P, P, P, P, LL, I, I, P, LL],
        "emu_gemm_store_ex": [P, P, I, I, I, I, LL, LL, P, P, LL, P, LL, I, P, P, P, I],
        "emu_convert_f32": [P, LL, I, P],
        "emu_target_shift": [P, LL, P, LL, I, I, I, P, LL, LL, LL, I, P, F, P],
        "emu_shift_fill": [I, P],
        "emu_exp_store_fixup": [P, LL, I, I, I, P, LL, LL, LL, P, P, P, P, P, F, P, LL, P, P, LL],
        "emu_scaled_colsum": [P, LL, I, I, I, P, P, P, I],
        "emu_exp_store_check": [I, P, LL, P, P],
        "emu_sweep_dz": [P, P, I, I, I, I, LL, LL, P, P, P, F, LL, P, P, P, P, P, P, LL, I, I],
        "emu_gemm_store": [P, P, I, I, I, I, LL, LL, P, LL, P, LL, I],
        "emu_coef": [LL, LL, F, F, I, I, LL, LL, LL, P, P, P, P, P, P, I, P, P, P],
        "emu_finalize": [LL, LL, F, F, I, I, LL, LL, LL, P, P, P, P, P, P, P, P, P, P, P],
        "emu_limit_to_active_rows": [I, I, I, I, I, P],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = I
    _lib = lib
    return lib


def ptr(t):
    return None if t is None else t.data_ptr()


class EmuLib(fake_lib.FakeLib):
    """FakeLib whose SIMT-only entry points compute for real (on host memory)."""

    def __init__(self):
        super().__init__()
        self.emu = load()

    def _ce_args(self, prob):
        return (prob.dtype, prob.logits, prob.ld, prob.n_rows, prob.vocab, prob.target, prob.ce_weight, prob.ignore_index,
                prob.label_smoothing, prob.lse_square_scale, prob.softcap, prob.reduction)

    def flce_b200_ce_forward(self, p, norm, rowstats, out, stream):
        self.calls.append("flce_b200_ce_forward")
        prob, fo = p._obj, out._obj
        self.structs.setdefault("flce_b200_ce_forward", []).append(prob)
        return self.emu.emu_ce_forward(*self._ce_args(prob), _addr(norm), _addr(rowstats), fo.lse, fo.target_prob, fo.loss_rows,
                                       fo.z_loss_rows, fo.correct_rows, fo.predicted_tokens, fo.scalars)

    def flce_b200_ce_backward(self, p, lse, norm, go, per_row, grad, ld_grad, scratch, stream):
        self.calls.append("flce_b200_ce_backward")
        return self.emu.emu_ce_backward(*self._ce_args(p._obj), _addr(lse), _addr(norm), _addr(go) or None, per_row, _addr(grad),
                                        ld_grad, _addr(scratch))

    def flce_b200_ce_forward_backward(self, p, norm, rowstats, out, grad, ld_grad, stream):
        # host restatement of the one-launch form: the two emulated passes, the second with an upstream gradient of 1
        self.calls.append("flce_b200_ce_forward_backward")
        prob, fo = p._obj, out._obj
        self.structs.setdefault("flce_b200_ce_forward_backward", []).append(prob)
        rc = self.emu.emu_ce_forward(*self._ce_args(prob), _addr(norm), _addr(rowstats), fo.lse, fo.target_prob, fo.loss_rows,
                                     fo.z_loss_rows, fo.correct_rows, fo.predicted_tokens, fo.scalars)
        if rc != 0:
            return rc
        scratch = (C.c_float * (3 * prob.n_rows))()
        return self.emu.emu_ce_backward(*self._ce_args(prob), fo.lse, _addr(norm), None, 0, _addr(grad), ld_grad,
                                        C.addressof(scratch))

    def flce_b200_ce_scale_gradient(self, grad, ld_grad, n_rows, vocab, dtype, go, per_row, stream):
        self.calls.append("flce_b200_ce_scale_gradient")
        import torch

        tdtype = {0: torch.bfloat16, 1: torch.float16, 2: torch.float32}[dtype]
        esize = 4 if dtype == 2 else 2
        raw = (C.c_char * (((n_rows - 1) * ld_grad + vocab) * esize)).from_address(_addr(grad))
        flat = torch.frombuffer(raw, dtype=tdtype)
        g = torch.as_strided(flat, (n_rows, vocab), (ld_grad, 1))
        scale = torch.frombuffer((C.c_char * (4 * (n_rows if per_row else 1))).from_address(_addr(go)), dtype=torch.float32)
        if per_row or float(scale[0]) != 1.0:
            g.copy_((g.float() * (scale[:, None] if per_row else scale[0])).to(tdtype))
        return 0

    def flce_b200_count(self, p, norm, stream):
        self.calls.append("flce_b200_count")
        prob = p._obj
        return self.emu.emu_count(prob.target, prob.n_rows, prob.ignore_index, prob.ce_weight, prob.vocab, prob.vocab_offset,
                                  float(prob.vocab_total), _addr(norm))

    def flce_b200_compact_rows(self, p, xc, tc, perm, active, stream):
        self.calls.append("flce_b200_compact_rows")
        prob = p._obj
        return self.emu.emu_compact_rows(prob.x, prob.ld_x, prob.hidden, prob.n_rows, prob.target, prob.ignore_index, _addr(xc),
                                         _addr(tc), _addr(perm), _addr(active))

    def flce_b200_compact_rows_rmsnorm(self, p, gamma, eps, offset, mode, xc, tc, perm, active, rstd, stream):
        self.calls.append("flce_b200_compact_rows_rmsnorm")
        prob = p._obj
        return self.emu.emu_compact_rows_rmsnorm(prob.x, prob.ld_x, prob.hidden, prob.n_rows, prob.target, prob.ignore_index,
                                                 prob.dtype, _addr(gamma), eps, offset, mode, _addr(xc), _addr(tc), _addr(perm),
                                                 _addr(active), _addr(rstd))

    def flce_b200_rmsnorm_partial_floats(self, hidden):
        return 8 * hidden

    def flce_b200_rmsnorm_scatter_backward(self, gy, ld_g, x, ld_x, dtype, n_rows, hidden, gamma, rstd, perm, active, offset, mode,
                                           gx, ld_gx, dgamma, partials, stream):
        self.calls.append("flce_b200_rmsnorm_scatter_backward")
        return self.emu.emu_rmsnorm_scatter_backward(_addr(gy), ld_g, _addr(x), ld_x, dtype, n_rows, hidden, _addr(gamma),
                                                     _addr(rstd), _addr(perm) or None, _addr(active) or None, offset, mode,
                                                     _addr(gx), ld_gx, _addr(dgamma), _addr(partials), min(8, n_rows))

    def flce_b200_scatter_rows(self, src, row_bytes, perm, active, n_rows, dst, stream):
        self.calls.append("flce_b200_scatter_rows")
        return self.emu.emu_scatter_rows(_addr(src), row_bytes, _addr(perm), _addr(active), n_rows, _addr(dst))

    def flce_b200_split_fp32(self, src, rows, cols, ld_src, dst, ld_dst, block_cols, pattern, n_blocks, dst_dtype, stream):
        self.calls.append("flce_b200_split_fp32")
        pat = (C.c_int * 8)(*[int(pattern[i]) for i in range(n_blocks)])
        return self.emu.emu_split_fp32(_addr(src), rows, cols, ld_src, _addr(dst), ld_dst, block_cols, C.addressof(pat), n_blocks,
                                       dst_dtype)

    def flce_b200_scale_gradient(self, data, n, dtype, scale, stream):
        self.calls.append("flce_b200_scale_gradient")
        return self.emu.emu_scale_inplace(_addr(data), n, {0: 0, 1: 1, 2: 2}[dtype], _addr(scale))


    def flce_b200_scaled_ce_rows(self, logits, ld, dtype, n_rows, vocab, target, ignore_index, temperature, nll, entropy, lse, stream):
        self.calls.append("flce_b200_scaled_ce_rows")
        return self.emu.emu_scaled_ce_rows(_addr(logits), ld, dtype, n_rows, vocab, _addr(target), ignore_index, temperature, _addr(nll),
                                           _addr(entropy), _addr(lse))

    def flce_b200_scaled_ce_grad(self, logits, ld, dtype, n_rows, vocab, target, ignore_index, temperature, lse, entropy, g_nll, g_ent,
                                 stream):
        self.calls.append("flce_b200_scaled_ce_grad")
        return self.emu.emu_scaled_ce_grad(_addr(logits), ld, dtype, n_rows, vocab, _addr(target), ignore_index, temperature, _addr(lse),
                                           _addr(entropy), _addr(g_nll) or None, _addr(g_ent) or None)

    def flce_b200_jsd_rows(self, student, ld_s, teacher, ld_t, dtype, n_rows, vocab, labels, ignore_index, beta, temperature, count,
                           fixed_count, loss_rows, stream):
        self.calls.append("flce_b200_jsd_rows")
        return self.emu.emu_jsd_rows(_addr(student), ld_s, _addr(teacher), ld_t, dtype, n_rows, vocab, _addr(labels) or None, ignore_index,
                                     beta, temperature, _addr(count) or None, fixed_count, _addr(loss_rows))

    # ---- the fused linear cross-entropy entry points: the library's epilogues and row kernels, its host sequence restated
    PAIR_ROWS = 256              # rows a CTA pair owns: granularity of the active-row limit on m-tiles

    @staticmethod
    def _matrix(addr, rows, cols, ld, dt):
        n_el = (rows - 1) * ld + cols
        buf = (C.c_char * (n_el * dt.itemsize)).from_address(addr)
        return torch.as_strided(torch.frombuffer(buf, dtype=dt, count=n_el), (rows, cols), (ld, 1))

    def _m_tile_limit(self, prob):
        if not prob.active_rows:
            return -1, prob.n_rows
        active = int(fake_lib._array(prob.active_rows, C.c_int32, 1)[0])
        pairs = (max(active, 0) + self.PAIR_ROWS - 1) // self.PAIR_ROWS
        return pairs * (self.PAIR_ROWS // 128), min(prob.n_rows, pairs * self.PAIR_ROWS)

    def flce_b200_forward_stats(self, p, rowstats, ws, ws_bytes, stream):
        self.calls.append("flce_b200_forward_stats")
        prob = p._obj
        self.structs.setdefault("flce_b200_forward_stats", []).append(prob)
        n, v = prob.n_rows, prob.vocab
        n_tiles = (v + 255) // 256
        nan = float("nan")                      # what the sweeps do not write stays poisoned, like real scratch memory
        planes = [torch.full((n_tiles, n), nan) for _ in range(4)]
        pidx = torch.zeros((n_tiles, n), dtype=torch.int32)
        fake_lib.float_array(_addr(rowstats) + 2 * n * 4, n)[:] = 0.0            # target-logit plane: the library memsets it
        limit, _ = self._m_tile_limit(prob)
        cap = float(prob.softcap)
        rc = self.emu.emu_sweep_stats(prob.x, prob.w, prob.dtype, n, v, prob.hidden, prob.ld_x, prob.ld_w, prob.target, prob.bias,
                                      prob.ce_weight, cap, prob.vocab_offset, planes[0].data_ptr(), planes[1].data_ptr(),
                                      planes[2].data_ptr(), planes[3].data_ptr(), pidx.data_ptr(), _addr(rowstats) + 2 * n * 4,
                                      None, 0, 0, limit, None, 0)
        self.emu.emu_merge_partials(n, n_tiles, planes[0].data_ptr(), planes[1].data_ptr(), planes[2].data_ptr(),
                                    planes[3].data_ptr(), pidx.data_ptr(), _addr(rowstats))
        return rc

    def flce_b200_forward_finalize(self, p, rowstats, norm, out, stream):
        self.calls.append("flce_b200_forward_finalize")
        prob, fo = p._obj, out._obj
        return self.emu.emu_finalize(prob.n_rows, prob.ignore_index, prob.label_smoothing, prob.lse_square_scale,
                                     int(prob.reduction == 0), prob.use_token_scaling, prob.vocab, prob.vocab_total, prob.vocab_offset,
                                     prob.target, prob.ce_weight, _addr(rowstats), _addr(norm), fo.lse, fo.target_prob, fo.loss_rows,
                                     fo.z_loss_rows, fo.correct_rows, fo.predicted_tokens, fo.scalars)

    def flce_b200_forward(self, p, norm, rowstats, out, ws, ws_bytes, stream):
        rc = self.flce_b200_count(p, norm, stream) or self.flce_b200_forward_stats(p, rowstats, ws, ws_bytes, stream) \
            or self.flce_b200_forward_finalize(p, rowstats, norm, out, stream)
        del self.calls[-3:]
        self.calls.append("flce_b200_forward")
        self.structs.setdefault("flce_b200_forward", []).append(p._obj)
        return rc

    def _backward_slabs(self, prob, budget):
        budget = budget or (1 << 30)
        max_cols = max(256, budget // (prob.n_rows * 2) // 256 * 256)
        n_slabs = (prob.vocab + max_cols - 1) // max_cols
        slab_cols = ((prob.vocab + n_slabs - 1) // n_slabs + 255) // 256 * 256
        return (prob.vocab + slab_cols - 1) // slab_cols, slab_cols

    def flce_b200_backward_plan(self, p, budget, n_slabs, slab_cols):
        self.calls.append("flce_b200_backward_plan")
        n_slabs._obj.value, slab_cols._obj.value = self._backward_slabs(p._obj, budget)
        return 0

    def flce_b200_backward(self, p, args, ws, ws_bytes, budget, stream):
        self.calls.append("flce_b200_backward")
        prob, a = p._obj, args._obj
        self.structs.setdefault("flce_b200_backward", []).append(a)
        tdt = {0: torch.bfloat16, 1: torch.float16}[prob.dtype]
        gdt = {0: torch.bfloat16, 1: torch.float16, 2: torch.float32}[a.grad_dtype]
        n, h, v = prob.n_rows, prob.hidden, prob.vocab
        px, px_cols, ld_px = (a.proj_x, a.proj_x_cols, a.ld_proj_x) if a.proj_x else (prob.x, h, prob.ld_x)
        pw, pw_cols, ld_pw = (a.proj_w, a.proj_w_cols, a.ld_proj_w) if a.proj_w else (prob.w, h, prob.ld_w)
        split = bool(a.split_logit_grad)
        PX = self._matrix(px, n, px_cols, ld_px, tdt).float()
        PW = self._matrix(pw, v, pw_cols, ld_pw, tdt).float()
        c = torch.zeros(3, n)
        self.emu.emu_coef(n, prob.ignore_index, prob.label_smoothing, prob.lse_square_scale, int(prob.reduction == 0),
                          prob.use_token_scaling, v, prob.vocab_total, prob.vocab_offset, prob.target, prob.ce_weight, a.lse,
                          a.target_prob, a.norm, a.grad_output, a.grad_output_per_row, c[0].data_ptr(), c[1].data_ptr(),
                          c[2].data_ptr())
        n_slabs, slab_cols = self._backward_slabs(prob, budget)
        first, last = (a.slab_begin, a.slab_end) if (a.slab_begin or a.slab_end) else (0, n_slabs)
        limit, row_limit = self._m_tile_limit(prob)
        k_rows = n
        if prob.active_rows:
            active = int(fake_lib._array(prob.active_rows, C.c_int32, 1)[0])
            k_rows = min(n, (max(active, 0) + 63) // 64 * 64)
        acc = self.__dict__.setdefault("_dx_acc", {})
        for s_i in range(first, last):
            v0 = s_i * slab_cols
            cols = min(slab_cols, v - v0)
            dz = torch.full((n, slab_cols), float("nan")).to(tdt)      # rows no tile covers stay poisoned
            dz_lo = torch.full((n, slab_cols), float("nan")).to(tdt) if split else None
            self.emu.emu_sweep_dz(prob.x, prob.w + v0 * prob.ld_w * 2, prob.dtype, n, cols, h, prob.ld_x, prob.ld_w, prob.target,
                                  prob.bias + v0 * 4 if prob.bias else None, prob.ce_weight + v0 * 4 if prob.ce_weight else None,
                                  float(prob.softcap), prob.vocab_offset + v0, a.lse, c[0].data_ptr(), c[1].data_ptr(),
                                  c[2].data_ptr(), dz.data_ptr(), None if dz_lo is None else dz_lo.data_ptr(), slab_cols, prob.dtype,
                                  limit)
            dzf = dz[:, :cols].float()
            lof = None if dz_lo is None else dz_lo[:, :cols].float()
            if a.grad_weight:
                gw = dzf[:k_rows].T @ PX[:k_rows]
                if split:
                    gw[:, :a.lo_cols_x] += lof[:k_rows].T @ PX[:k_rows, :a.lo_cols_x]
                self._matrix(a.grad_weight, v, px_cols, px_cols, gdt)[v0:v0 + cols] = gw.to(gdt)
            if a.grad_input:
                part = dzf[:row_limit] @ PW[v0:v0 + cols]
                if split:
                    part[:, :a.lo_cols_w] += lof[:row_limit] @ PW[v0:v0 + cols, :a.lo_cols_w]
                acc[a.grad_input] = part if s_i == 0 else acc[a.grad_input] + part
                if s_i == n_slabs - 1:
                    self._matrix(a.grad_input, n, pw_cols, pw_cols, gdt)[:row_limit] = acc.pop(a.grad_input).to(gdt)
            if a.grad_bias:
                gb = dzf[:k_rows].sum(0) + (0 if lof is None else lof[:k_rows].sum(0))
                fake_lib.float_array(a.grad_bias + v0 * 4, cols)[:] = gb.numpy()
        return 0

    # ---- single-sweep mode: the host sequence of flce_b200_forward_backward restated around the emulated pieces
    CHUNK_ROWS = 256             # rows per token chunk here (the library sizes chunks from a byte budget, in multiples of 256)

    def flce_b200_forward_backward(self, p, args, ws, ws_bytes, budget, stream):
        self.calls.append("flce_b200_forward_backward")
        prob, a = p._obj, args._obj
        self.structs.setdefault("flce_b200_forward_backward", []).append(prob)
        fo = a.out.contents
        tdt = {0: torch.bfloat16, 1: torch.float16}[prob.dtype]
        gdt = {0: torch.bfloat16, 1: torch.float16, 2: torch.float32}[a.grad_dtype]
        gfmt = a.grad_dtype
        n, h, v = prob.n_rows, prob.hidden, prob.vocab
        smoothing = prob.label_smoothing > 0
        cap = float(prob.softcap)
        exp_ok = not (smoothing and cap > 0) and not a.grad_bias and prob.dtype == 0
        if a.store_mode == 2 and not exp_ok:
            return 2
        sharded = prob.vocab != prob.vocab_total or prob.vocab_offset != 0
        if sharded and not (a.exchange_shift and a.exchange_rowstats and a.after_grad_input):
            return 2
        from liger_kernel_b200 import _lib as real_lib
        exp_store = exp_ok and a.store_mode != 1
        self.store_modes = getattr(self, "store_modes", []) + ["exp" if exp_store else "logits"]
        if not a.norm_given:
            self.emu.emu_count(prob.target, n, prob.ignore_index, prob.ce_weight, v, prob.vocab_offset, float(prob.vocab_total), a.norm)
        active = int(fake_lib._array(prob.active_rows, C.c_int32, 1)[0]) if prob.active_rows else None
        active_ptr = prob.active_rows if prob.active_rows else None
        W16 = self._matrix(prob.w, v, h, prob.ld_w, tdt)
        Wt = W16.t().contiguous()                                   # [h, v]: B operand of grad_input, K (= vocabulary) contiguous
        n_tiles = (v + 255) // 256
        ld_slab = (v + 63) // 64 * 64
        nan = float("nan")
        dw_acc = torch.full((v, h), nan)
        gb = torch.zeros(v)
        shift = torch.full((n,), nan)
        w_sum, x_sum = torch.full((h,), nan), torch.full((h,), nan)
        scratch = torch.full((32, h), nan)
        if exp_store:
            self.emu.emu_target_shift(prob.x, prob.ld_x, prob.w, prob.ld_w, prob.dtype, n, h, prob.target, prob.ignore_index, v,
                                      prob.vocab_offset, int(sharded), prob.bias, cap, shift.data_ptr())
            if sharded:
                real_lib.EXCHANGE_SHIFT_FN(a.exchange_shift)(a.exchange_user, shift.data_ptr(), n)
                self.emu.emu_shift_fill(n, shift.data_ptr())
            if smoothing and a.grad_input:
                self.emu.emu_scaled_colsum(prob.w, prob.ld_w, v, h, prob.dtype, prob.ce_weight, scratch.data_ptr(), w_sum.data_ptr(), 0)
        off = lambda base, rows, size: (base + rows * size) if base else None      # noqa: E731
        chunks = list(range(0, n, self.CHUNK_ROWS))
        for r0 in chunks:
            first, last = r0 == chunks[0], r0 == chunks[-1]
            rows = min(self.CHUNK_ROWS, n - r0)
            live = rows if active is None else min(rows, max(0, active - r0))
            pairs = (live + self.PAIR_ROWS - 1) // self.PAIR_ROWS
            limit = -1 if active is None else pairs * (self.PAIR_ROWS // 128)
            row_limit = rows if active is None else min(rows, pairs * self.PAIR_ROWS)
            k_rows = rows if active is None else min(rows, (live + 63) // 64 * 64)
            x_c = prob.x + r0 * prob.ld_x * 2
            t_c = prob.target + r0 * 8
            planes = [torch.full((n_tiles, rows), nan) for _ in range(4)]
            pidx = torch.zeros((n_tiles, rows), dtype=torch.int32)
            stats = torch.full((6, rows), nan)
            stats[2] = 0.0
            slab = torch.full((rows, ld_slab), nan).to(tdt)        # what the sweep does not write stays poisoned
            self.emu.emu_sweep_stats(x_c, prob.w, prob.dtype, rows, v, h, prob.ld_x, prob.ld_w, t_c, prob.bias, prob.ce_weight, cap,
                                     prob.vocab_offset, planes[0].data_ptr(), planes[1].data_ptr(), planes[2].data_ptr(),
                                     planes[3].data_ptr(), pidx.data_ptr(), stats[2].data_ptr(), slab.data_ptr(), ld_slab,
                                     prob.dtype, limit, shift[r0:].data_ptr() if exp_store else None, prob.ignore_index)
            self.emu.emu_merge_partials(rows, n_tiles, planes[0].data_ptr(), planes[1].data_ptr(), planes[2].data_ptr(),
                                        planes[3].data_ptr(), pidx.data_ptr(), stats.data_ptr())
            if sharded:
                real_lib.EXCHANGE_ROWSTATS_FN(a.exchange_rowstats)(a.exchange_user, stats.data_ptr(), rows, r0)
            self.emu.emu_finalize(rows, prob.ignore_index, prob.label_smoothing, prob.lse_square_scale, int(prob.reduction == 0),
                                  prob.use_token_scaling, v, prob.vocab_total, prob.vocab_offset, t_c, prob.ce_weight,
                                  stats.data_ptr(), a.norm, off(fo.lse, r0, 4), off(fo.target_prob, r0, 4), off(fo.loss_rows, r0, 4),
                                  off(fo.z_loss_rows, r0, 4), off(fo.correct_rows, r0, 4), off(fo.predicted_tokens, r0, 8), None)
            c = torch.zeros(3, rows)
            self.emu.emu_coef(rows, prob.ignore_index, prob.label_smoothing, prob.lse_square_scale, int(prob.reduction == 0),
                              prob.use_token_scaling, v, prob.vocab_total, prob.vocab_offset, t_c, prob.ce_weight, off(fo.lse, r0, 4),
                              off(fo.target_prob, r0, 4), a.norm, None, 0, c[0].data_ptr(), c[1].data_ptr(), c[2].data_ptr())
            alpha = torch.full((rows,), nan)
            xs = torch.full((rows, h), nan).to(tdt)
            if exp_store:
                redo = self.emu.emu_exp_store_check(rows, t_c, prob.ignore_index, off(fo.lse, r0, 4), shift[r0:].data_ptr())
                self.redo_chunks = getattr(self, "redo_chunks", 0) + int(redo)
                if redo:      # the gated repeat of sweep 1 with the reference points on the log-sum-exp
                    tl = torch.zeros(rows)
                    self.emu.emu_sweep_stats(x_c, prob.w, prob.dtype, rows, v, h, prob.ld_x, prob.ld_w, t_c, prob.bias,
                                             prob.ce_weight, cap, prob.vocab_offset, planes[0].data_ptr(), planes[1].data_ptr(),
                                             planes[2].data_ptr(), planes[3].data_ptr(), pidx.data_ptr(), tl.data_ptr(),
                                             slab.data_ptr(), ld_slab, prob.dtype, limit, shift[r0:].data_ptr(), prob.ignore_index)
                self.emu.emu_exp_store_fixup(x_c, prob.ld_x, h, prob.dtype, rows, t_c, prob.ignore_index, v, prob.vocab_offset,
                                             off(fo.lse, r0, 4),
                                             shift[r0:].data_ptr(), stats[2].data_ptr(), c[0].data_ptr(), c[2].data_ptr(), cap,
                                             slab.data_ptr(), ld_slab, alpha.data_ptr(), xs.data_ptr(), h)
                if smoothing and a.grad_weight:
                    self.emu.emu_scaled_colsum(x_c, prob.ld_x, rows, h, prob.dtype, c[1].data_ptr(), scratch.data_ptr(),
                                               x_sum.data_ptr(), int(not first))
            else:
                self.emu.emu_dz_inplace(slab.data_ptr(), ld_slab, rows, v, prob.dtype, t_c, prob.vocab_offset, off(fo.lse, r0, 4),
                                        c[0].data_ptr(), c[1].data_ptr(), c[2].data_ptr(), prob.ce_weight,
                                        1.0 / cap if cap > 0 else 0.0, active_ptr, r0)
            def grad_input_part():
                if a.grad_input and row_limit > 0:
                    # grad_input[chunk] = dZ . W through the library's store epilogue (per-row factor and rank-1 term in exp-store form)
                    gi = a.grad_input + r0 * h * (4 if gfmt == 2 else 2)
                    self.emu.emu_gemm_store_ex(slab.data_ptr(), Wt.data_ptr(), prob.dtype, row_limit, h, v, ld_slab, v, None, None, 0,
                                               gi, h, gfmt, alpha.data_ptr() if exp_store else None,
                                               c[1].data_ptr() if (exp_store and smoothing) else None,
                                               w_sum.data_ptr() if (exp_store and smoothing) else None, 0)
                if sharded and a.grad_input:
                    real_lib.AFTER_GRAD_INPUT_FN(a.after_grad_input)(a.exchange_user, a.grad_input + r0 * h * (4 if gfmt == 2 else 2),
                                                                     rows, r0)

            def grad_weight_part():
                if a.grad_weight:
                    X16 = xs if exp_store else self._matrix(x_c, rows, h, prob.ld_x, tdt)
                    At = slab[:k_rows, :v].t().contiguous()             # [v, k_rows]
                    Bt = X16[:k_rows].t().contiguous()                  # [h, k_rows]
                    kk = k_rows
                    if kk == 0:                                         # nothing accumulated: the kernel's k_blocks == 0 path
                        At, Bt, kk = torch.zeros(v, 8).to(tdt), torch.zeros(h, 8).to(tdt), 8
                    r1 = exp_store and smoothing and last
                    # one chunk: written once in the final dtype; several: first stores fp32, the others add, 16-bit converted at the end
                    direct = len(chunks) == 1 and gfmt != 2
                    acc_t = self._matrix(a.grad_weight, v, h, h, torch.float32) if gfmt == 2 else dw_acc
                    self.emu.emu_gemm_store_ex(At.data_ptr(), Bt.data_ptr(), prob.dtype, v, h, kk, kk, kk, None,
                                               None if direct else acc_t.data_ptr(), h, a.grad_weight if direct else None, h, prob.dtype,
                                               None, prob.ce_weight if r1 else None, x_sum.data_ptr() if r1 else None,
                                               int(not direct and not first))
                    if last and not direct and gfmt != 2:
                        self.emu.emu_convert_f32(dw_acc.data_ptr(), v * h, prob.dtype, a.grad_weight)

            if last and a.after_grad_weight:          # the library's order when a caller sums grad_weight over token shards
                grad_weight_part()
                real_lib.AFTER_GRAD_WEIGHT_FN(a.after_grad_weight)(a.after_grad_weight_user)
                grad_input_part()
            else:
                grad_input_part()
                grad_weight_part()
            if a.grad_bias:
                self.emu.emu_colsum(slab.data_ptr(), ld_slab, rows, v, prob.dtype, gb.data_ptr(), int(r0 != 0), active_ptr, r0)
        if a.grad_bias:
            fake_lib.float_array(a.grad_bias, v)[:] = gb.numpy()
        if fo.scalars:
            self.emu.emu_reduce_rows(n, fo.loss_rows, fo.z_loss_rows, fo.correct_rows, a.norm, fo.scalars)
        return 0

    # ---- scaled cross-entropy on the two sweeps: the library's epilogues tile by tile, its slab loop restated here
    SCE_SLAB_COLS = 256          # small slabs so that the slab offsets are exercised

    def flce_b200_sce_workspace_bytes(self, p, phase, budget):
        self.calls.append("flce_b200_sce_workspace_bytes")
        prob = p._obj
        n_tiles = (prob.vocab + 255) // 256
        return 4 * (3 * n_tiles * prob.n_rows + prob.n_rows) + 1024

    def flce_b200_sce_forward(self, p, nll, entropy, lse, ws, ws_bytes, stream):
        self.calls.append("flce_b200_sce_forward")
        prob = p._obj
        n_tiles = (prob.vocab + 255) // 256
        planes = torch.zeros(3 * n_tiles * prob.n_rows)
        target_logit = torch.zeros(prob.n_rows)
        return self.emu.emu_sce_forward(prob.x, prob.w, prob.dtype, prob.n_rows, prob.vocab, prob.hidden, prob.ld_x, prob.ld_w,
                                        prob.target, prob.ignore_index, prob.temperature, planes.data_ptr(), target_logit.data_ptr(),
                                        _addr(nll), _addr(entropy), _addr(lse))

    def flce_b200_sce_backward(self, p, lse, entropy, g_nll, g_ent, grad_dtype, grad_input, grad_weight, ws, ws_bytes, budget, stream):
        self.calls.append("flce_b200_sce_backward")
        prob = p._obj
        tdt = {0: torch.bfloat16, 1: torch.float16}[prob.dtype]
        gdt = {0: torch.bfloat16, 1: torch.float16, 2: torch.float32}[grad_dtype]
        m, h, v = prob.n_rows, prob.hidden, prob.vocab

        def matrix(addr, rows, cols, ld, dt):
            n_el = (rows - 1) * ld + cols
            buf = (C.c_char * (n_el * dt.itemsize)).from_address(addr)
            return torch.as_strided(torch.frombuffer(buf, dtype=dt, count=n_el), (rows, cols), (ld, 1))

        x = matrix(prob.x, m, h, prob.ld_x, tdt).float()
        w = matrix(prob.w, v, h, prob.ld_w, tdt)
        gx = torch.zeros(m, h)
        for v0 in range(0, v, self.SCE_SLAB_COLS):
            cols = min(self.SCE_SLAB_COLS, v - v0)
            dz = torch.zeros((m, self.SCE_SLAB_COLS), dtype=tdt)
            w_slab = w[v0:v0 + cols]
            self.emu.emu_sce_sweep_dz(prob.x, w_slab.data_ptr(), prob.dtype, m, cols, h, prob.ld_x, prob.ld_w, prob.target,
                                      prob.ignore_index, prob.temperature, v0, _addr(lse), _addr(entropy), _addr(g_nll) or None,
                                      _addr(g_ent) or None, dz.data_ptr(), self.SCE_SLAB_COLS, prob.dtype)
            dzf = dz[:, :cols].float()
            if _addr(grad_weight):
                matrix(_addr(grad_weight), v, h, h, gdt)[v0:v0 + cols] = (dzf.T @ x).to(gdt)
            gx += dzf @ w_slab.float()
        if _addr(grad_input):
            matrix(_addr(grad_input), m, h, h, gdt).copy_(gx.to(gdt))
        return 0

    def flce_b200_gemm_accumulate(self, a, b, acc, out, m, n, k, ld_a, ld_b, ld_acc, ld_out, ab_dtype, out_dtype, a_mn_major,
                                  b_mn_major, cta_pair, stream):
        """The tensor-core GEMM replaced by torch on host memory: 16-bit operands, fp32 accumulation, the library's
        layouts (K-major [rows, k] or MN-major [k, rows]) and its two outputs."""
        self.calls.append("flce_b200_gemm_accumulate")
        tdt = {0: torch.bfloat16, 1: torch.float16}[ab_dtype]

        def matrix(addr, rows, cols, ld, dt):       # [rows, cols] view with row pitch ld
            n_el = (rows - 1) * ld + cols
            buf = (C.c_char * (n_el * dt.itemsize)).from_address(addr)
            flat = torch.frombuffer(buf, dtype=dt, count=n_el)
            return torch.as_strided(flat, (rows, cols), (ld, 1))

        A = matrix(_addr(a), k, m, ld_a, tdt).T if a_mn_major else matrix(_addr(a), m, k, ld_a, tdt)
        B = matrix(_addr(b), k, n, ld_b, tdt).T if b_mn_major else matrix(_addr(b), n, k, ld_b, tdt)
        v = A.float() @ B.float().T
        if _addr(acc):
            ACC = matrix(_addr(acc), m, n, ld_acc, torch.float32)
            v = v + ACC
            ACC.copy_(v)
        if _addr(out):
            odt = {0: torch.bfloat16, 1: torch.float16, 2: torch.float32}[out_dtype]
            matrix(_addr(out), m, n, ld_out, odt).copy_(v.to(odt))
        return 0


@contextlib.contextmanager
def installed(monkeypatch):
    """Like fake_lib.installed, with the SIMT-only entry points computing through the emulation."""
    import liger_kernel_b200.ops.cross_entropy as ce
    import liger_kernel_b200.ops.fused_linear_cross_entropy as fl
    import liger_kernel_b200.sharded as sh

    lib = EmuLib()
    for mod in (fl, ce, sh):
        monkeypatch.setattr(mod, "lib", lib)
    monkeypatch.setattr(fl, "_stream", lambda device: None)
    monkeypatch.setattr(fl, "_device_guard", lambda device: contextlib.nullcontext())
    monkeypatch.setattr(fl, "_require_cuda", lambda t: None)
    yield lib
