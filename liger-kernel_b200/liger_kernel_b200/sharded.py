"""FLCE across the GPUs of one box: token-sharded and vocabulary-sharded operators.

One process per GPU, collectives through ``torch.distributed`` (NCCL on GPUs).  Nothing in here reads a
peer's memory: the collectives land in local HBM and the kernels only ever see local pointers.

Token-sharded (data parallel; the reference leaves this to DDP/FSDP, ``README.md:117``): every rank holds its
own rows of X / target and the whole W.  Exchanges: the normalisers (count of non-ignored rows, class-weight
sum) before the per-row losses are formed, the scalar loss, and grad_weight (summed).  With mean / sum reduction
and 16-bit operands the gradients are formed in forward (``ops/fused_linear_cross_entropy.py``, single-sweep
mode) with the all-reduced normalisers, and grad_weight is all-reduced right after the sweep.  Optionally
(``OVERLAP_GRAD_WEIGHT``) the last token chunk forms grad_weight first, the all-reduce starts on a side stream as
soon as that GEMM is done, and the chunk's grad_input GEMM runs beside it on the SMs it leaves free.  Otherwise
(``reduction="none"``, fp32) backward recomputes the logits and all-reduces grad_weight after it.

Vocabulary-sharded (tensor parallel; the math and collective pattern follow the reference's
``ops/vocab_parallel_cross_entropy.py:235-303``): every rank holds rows ``[vocab_start, vocab_start+V_r)`` of W and
the whole X / target (global class ids).  Exchanges: one all-gather of the ``[6, N]`` per-row statistics after
sweep 1 (max, sum-exp, target logit, logit sum, arg-max value and index) merged locally in rank order — instead
of the reference's all-reduce(MAX) + 2 x all-reduce(SUM) — and an all-reduce(SUM) of the partial grad_input.
Label smoothing uses the global vocabulary size.

The local computation is reached through a small backend object so that the exchange logic can be exercised
on CPU ranks (gloo) with a stand-in backend in the tests; the default backend is the CUDA library.
"""

from __future__ import annotations

import ctypes as C
import os

import torch
import torch.distributed as dist

from . import _lib
from ._lib import check, lib
from .ops import fused_linear_cross_entropy as _op


class CudaBackend:
    """Local FLCE pieces on the current GPU through libflce_b200.so."""

    def prepare(self, x, w, target, bias, ce_weight, ignore_index, lse_square_scale, label_smoothing, reduction, softcap,
                use_token_scaling, vocab_total=None, vocab_offset=0, want_argmax=False, allow_compact=False):
        return _op._Prepared(x, w, target, bias, ce_weight, ignore_index, lse_square_scale, label_smoothing, reduction,
                             softcap, use_token_scaling, vocab_total=vocab_total, vocab_offset=vocab_offset,
                             want_argmax=want_argmax, allow_compact=allow_compact)

    def single_sweep(self, prep, norm, need_input, need_weight, after_grad_weight=None, reserve_sms=0, shard_hooks=None,
                     grad_dtype=None):
        """Loss rows / scalars and the gradients for an upstream gradient of 1, with the given (global) normalisers.
        grad_input comes back in the compact row order of ``prep`` (``prep.rows_to_token_order`` undoes it)."""
        out, _, gx, gw, _ = _op.flce_single_sweep_device(prep, need_input, need_weight, False, norm_in=norm,
                                                         after_grad_weight=after_grad_weight, reserve_sms=reserve_sms,
                                                         shard_hooks=shard_hooks, grad_dtype=grad_dtype)
        return _op._results_to_token_order(prep, out), gx, gw

    def count(self, prep):
        norm = torch.empty(4, dtype=torch.float32, device=prep.device)
        with _op._device_guard(prep.device):
            check(lib.flce_b200_count(C.byref(prep.problem), _op._ptr(norm), _op._stream(prep.device)))
        return norm

    def forward_stats(self, prep):
        rowstats = torch.empty((_lib.ROWSTAT_PLANES, prep.n_rows), dtype=torch.float32, device=prep.device)
        with _op._device_guard(prep.device):
            ws = prep.workspace(_lib.PHASE_FORWARD)
            check(lib.flce_b200_forward_stats(C.byref(prep.problem), _op._ptr(rowstats), _op._ptr(ws), ws.numel(),
                                              _op._stream(prep.device)))
        return rowstats

    def finalize(self, prep, rowstats, norm):
        out = _op._forward_outputs(prep)
        fo = _op._as_forward_out(out)
        with _op._device_guard(prep.device):
            check(lib.flce_b200_forward_finalize(C.byref(prep.problem), _op._ptr(rowstats), _op._ptr(norm), C.byref(fo),
                                                 _op._stream(prep.device)))
        return out

    def backward(self, prep, lse, target_prob, norm, grad_output, need_input, need_weight, grad_dtype=None, slab_hook=None):
        gx, gw, _ = _op.flce_backward_device(prep, lse, target_prob, norm, grad_output, need_input, need_weight, False,
                                             grad_dtype=grad_dtype, slab_hook=slab_hook)
        return gx, gw


def merge_rowstats(gathered: torch.Tensor) -> torch.Tensor:
    """Merge per-rank row statistics ``[G, 6, N]`` (ranks ordered by vocabulary offset) into ``[6, N]``.

    max: max over ranks; sum-exp: rescaled to the global max; target logit and logit sum: added (only the owner rank
    has a non-zero target logit); arg-max: largest value, lowest rank (= lowest class id) on ties."""
    m_r, d_r = gathered[:, 0], gathered[:, 1]
    m = m_r.max(dim=0).values
    d = (d_r * torch.exp(m_r - m[None, :])).sum(dim=0)
    xy = gathered[:, 2].sum(dim=0)
    ss = gathered[:, 3].sum(dim=0)
    best_val, best_rank = gathered[:, 4].max(dim=0)  # torch returns the first (lowest-rank) maximum
    idx_bits = gathered[:, 5].gather(0, best_rank[None, :])[0]
    return torch.stack([m, d, xy, ss, best_val, idx_bits], dim=0).contiguous()


def _world(group):
    return dist.get_world_size(group) if dist.is_initialized() else 1


# Optional device timing of the collectives: set to a list and every collective issued by the operators below appends
# (name, start_event, end_event), recorded on the stream that issues it (a benchmark reads them after a synchronise).
COLLECTIVE_EVENTS = None


class _timed:
    def __init__(self, name):
        self.name = name

    def __enter__(self):
        if COLLECTIVE_EVENTS is not None and torch.cuda.is_available():
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()
        return self

    def __exit__(self, *exc):
        if COLLECTIVE_EVENTS is not None and torch.cuda.is_available():
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            COLLECTIVE_EVENTS.append((self.name, self.start, end))


# SMs the last grad_input GEMM of a token-sharded call leaves to the grad_weight all-reduce that runs beside it
RESERVE_SMS_FOR_COLLECTIVE = 20
# Whether a sharded call's big collective starts beside the GEMM that follows it (side stream, SMs reserved) or is issued on
# the compute stream with every SM to itself.  Measured on 2 GPUs, NCCL beside one of this library's GEMMs moves 40 - 80 GB/s
# against 240 GB/s alone, so hiding pays only where the GEMM window is long:
# * vocabulary shards: each chunk's partial grad_input (a few hundred MB) rides behind that chunk's grad_weight GEMM: on by
#   default (LIGER_B200_SHARDED_OVERLAP=0 turns it off);
# * token shards: grad_weight (as large as the weight) would have only the last chunk's grad_input GEMM to hide behind: off by
#   default (LIGER_B200_SHARDED_OVERLAP_GRAD_WEIGHT=1 turns it on).
OVERLAP_COLLECTIVES = os.environ.get("LIGER_B200_SHARDED_OVERLAP", "1") == "1"
OVERLAP_GRAD_WEIGHT = os.environ.get("LIGER_B200_SHARDED_OVERLAP_GRAD_WEIGHT", "0") == "1"


def new_group_for_collectives_beside_gemm(ranks=None, max_ctas=16, **kwargs):
    """A second NCCL process group whose kernels use at most ``max_ctas`` thread blocks, for calls whose collectives run
    beside a GEMM that left them ``RESERVE_SMS_FOR_COLLECTIVE`` SMs (pass it as ``group=`` to the vocabulary-sharded
    operator, or to the token-sharded one when ``OVERLAP_GRAD_WEIGHT`` is on).  A collective that has the GPU to itself
    (grad_weight of token shards, by default) should stay on a group without that limit: measured on 2 B200s the same
    1 GB all-reduce moves 218 GB/s through 16 blocks.  One call issues all its collectives on one group, so no two
    communicators ever have kernels in flight at the same time."""
    options = dist.ProcessGroupNCCL.Options()
    options.config.max_ctas = int(max_ctas)
    return dist.new_group(ranks=ranks, backend="nccl", pg_options=options, **kwargs)


class _TokenSharded(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, target, group, backend, overlap, kw):
        recording = kw.get("recording", True)
        needs = (recording and ctx.needs_input_grad[0], recording and ctx.needs_input_grad[1])
        single = hasattr(backend, "single_sweep") and _op._use_single_sweep(kw["reduction"], needs, x.dtype)
        ctx.stored = None
        world = _world(group)
        if single:
            prep = backend.prepare(x.detach(), w.detach(), target, None, kw.get("ce_weight"), kw["ignore_index"],
                                   kw["lse_square_scale"], kw["label_smoothing"], kw["reduction"], kw["softcap"], False,
                                   allow_compact=True)
        else:
            prep = backend.prepare(x.detach(), w.detach(), target, None, kw.get("ce_weight"), kw["ignore_index"],
                                   kw["lse_square_scale"], kw["label_smoothing"], kw["reduction"], kw["softcap"], False)
        norm = backend.count(prep)
        if world > 1:
            counts = norm[:2].clone()          # norm[2] (sum of all class weights) is the same on every rank
            with _timed("all_reduce normalisers"):
                dist.all_reduce(counts, group=group)
            norm = torch.cat([counts, norm[2:]])
        if single:
            pending = []
            hook = None
            comm = None
            if world > 1 and needs[1] and OVERLAP_GRAD_WEIGHT:
                comm = torch.cuda.Stream(device=prep.device) if prep.device.type == "cuda" else None

                def hook(gw):
                    if comm is None:             # host tensors (tests on gloo ranks): nothing to overlap with
                        dist.all_reduce(gw, group=group)
                        return
                    done = torch.cuda.Event()
                    done.record()
                    comm.wait_event(done)
                    with torch.cuda.stream(comm):
                        with _timed("all_reduce grad_weight (beside the last grad_input GEMM)"):
                            work = dist.all_reduce(gw, group=group, async_op=True)
                            work.wait()              # comm waits for the collective; the compute stream does so in backward
                        pending.append(work)

            out, gx, gw = backend.single_sweep(prep, norm, needs[0], needs[1], after_grad_weight=hook,
                                               reserve_sms=RESERVE_SMS_FOR_COLLECTIVE if comm is not None else 0)
            if world > 1 and needs[1] and hook is None:
                with _timed("all_reduce grad_weight (after the sweep)"):
                    dist.all_reduce(gw, group=group)
            gx = prep.rows_to_token_order(gx)
            ctx.stored = (gx, gw, pending)
            ctx.hidden = prep.hidden
            ctx.in_dtypes = (x.dtype, w.dtype)
            ctx.group = group
            loss = out["scalars"][0].clone()
            if world > 1:
                with _timed("all_reduce loss"):
                    dist.all_reduce(loss, group=group)
            ctx.comm = comm
            return loss
        out = backend.finalize(prep, backend.forward_stats(prep), norm)
        ctx.saved = (prep, out["lse"], out["target_prob"], norm)
        ctx.group, ctx.backend, ctx.overlap = group, backend, overlap
        ctx.in_dtypes = (x.dtype, w.dtype)
        if kw["reduction"] == "none":
            return out["loss_rows"]
        loss = out["scalars"][0].clone()
        if _world(group) > 1:
            dist.all_reduce(loss, group=group)
        return loss

    @staticmethod
    def backward(ctx, grad_output):
        if ctx.stored is not None:
            gx, gw, pending = ctx.stored
            ctx.stored = None
            if ctx.comm is not None:             # the compute stream waits for the all-reduce of grad_weight
                torch.cuda.current_stream().wait_stream(ctx.comm)
            dev = (gx if gx is not None else gw).device
            go = grad_output.detach().to(device=dev, dtype=torch.float32).reshape(1)
            gx = _op.scale_gradient_(gx, go)
            gw = _op.scale_gradient_(gw, go)
            h = ctx.hidden
            gx = None if gx is None else gx[:, :h].to(ctx.in_dtypes[0])
            gw = None if gw is None else gw[:, :h].to(ctx.in_dtypes[1])
            return gx, gw, None, None, None, None, None
        prep, lse, prob, norm = ctx.saved
        group, backend = ctx.group, ctx.backend
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        world = _world(group)
        hook = None
        pending = []
        if world > 1 and need_w and ctx.overlap and prep.device.type == "cuda":
            comm = torch.cuda.Stream(device=prep.device)

            def hook(first_row, last_row, gw):
                ev = torch.cuda.Event()
                ev.record()
                comm.wait_event(ev)
                with torch.cuda.stream(comm):
                    pending.append(dist.all_reduce(gw[first_row:last_row], group=group, async_op=True))

        gx, gw = backend.backward(prep, lse, prob, norm, grad_output, need_x, need_w, slab_hook=hook)
        if world > 1 and need_w:
            if hook is None:
                with _timed("all_reduce grad_weight (after backward)"):
                    dist.all_reduce(gw, group=group)
            else:
                for work in pending:
                    work.wait()
                torch.cuda.current_stream(prep.device).wait_stream(comm)
        h = prep.hidden
        gx = None if gx is None else gx[:, :h].to(ctx.in_dtypes[0])
        gw = None if gw is None else gw[:, :h].to(ctx.in_dtypes[1])
        return gx, gw, None, None, None, None, None


def _merge_rowstats_in_place(stats, world, group):
    planes, n = stats.shape
    gathered = torch.empty((world * planes, n), dtype=stats.dtype, device=stats.device)
    with _timed("all_gather row statistics"):
        dist.all_gather_into_tensor(gathered, stats.contiguous(), group=group)
    stats.copy_(merge_rowstats(gathered.view(world, planes, n)))


class _VocabSharded(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_shard, target, vocab_start, vocab_total, group, backend, kw):
        recording = kw.get("recording", True)
        needs = (recording and ctx.needs_input_grad[0], recording and ctx.needs_input_grad[1])
        world = _world(group)
        ctx.stored = None
        if hasattr(backend, "single_sweep") and _op._use_single_sweep(kw["reduction"], needs, x.dtype):
            # Gradients formed in forward on every shard: the three exchanges happen inside the sweep, between launches
            # (reference points: max over shards; row statistics per token chunk: all-gather + merge; partial grad_input
            # of a chunk: summed over the shards on a side stream while the chunk's grad_weight GEMM runs).
            prep = backend.prepare(x.detach(), w_shard.detach(), target, None, None, kw["ignore_index"], kw["lse_square_scale"],
                                   kw["label_smoothing"], kw["reduction"], kw["softcap"], False, vocab_total=vocab_total,
                                   vocab_offset=vocab_start, want_argmax=True, allow_compact=True)
            norm = backend.count(prep)          # targets are replicated: identical on every rank
            on_gpu = prep.device.type == "cuda"
            comm = torch.cuda.Stream(device=prep.device) if (on_gpu and world > 1 and OVERLAP_COLLECTIVES) else None

            def exchange_shift(shift):
                if world > 1:
                    with _timed("all_reduce(max) reference points"):
                        dist.all_reduce(shift, op=dist.ReduceOp.MAX, group=group)

            def exchange_rowstats(stats, first_row):
                if world > 1:
                    _merge_rowstats_in_place(stats, world, group)

            def after_grad_input(gx_chunk, first_row):
                if world == 1:
                    return
                if comm is None:
                    dist.all_reduce(gx_chunk, group=group)
                    return
                done = torch.cuda.Event()
                done.record()
                comm.wait_event(done)
                with torch.cuda.stream(comm):
                    with _timed("all_reduce grad_input chunk (beside the grad_weight GEMM)"):
                        dist.all_reduce(gx_chunk, group=group, async_op=True).wait()

            hooks = dict(exchange_shift=exchange_shift, exchange_rowstats=exchange_rowstats, after_grad_input=after_grad_input)
            out, gx, gw = backend.single_sweep(prep, norm, needs[0], needs[1], shard_hooks=hooks, grad_dtype=torch.float32,
                                               reserve_sms=RESERVE_SMS_FOR_COLLECTIVE if comm is not None else 0)
            if comm is not None:
                torch.cuda.current_stream(prep.device).wait_stream(comm)
            gx = prep.rows_to_token_order(gx)
            ctx.stored = (gx, gw)
            ctx.hidden = prep.hidden
            ctx.in_dtypes = (x.dtype, w_shard.dtype)
            ctx.extra = dict(predicted_tokens=out["predicted_tokens"], z_loss=out["scalars"][1])
            return out["scalars"][0].clone()
        prep = backend.prepare(x.detach(), w_shard.detach(), target, None, None, kw["ignore_index"], kw["lse_square_scale"],
                               kw["label_smoothing"], kw["reduction"], kw["softcap"], False, vocab_total=vocab_total,
                               vocab_offset=vocab_start, want_argmax=True)
        norm = backend.count(prep)              # targets are replicated: identical on every rank
        stats = backend.forward_stats(prep)
        world = _world(group)
        if world > 1:
            planes, n = stats.shape
            gathered = torch.empty((world * planes, n), dtype=stats.dtype, device=stats.device)
            with _timed("all_gather row statistics"):
                dist.all_gather_into_tensor(gathered, stats.contiguous(), group=group)
            stats = merge_rowstats(gathered.view(world, planes, n))
        out = backend.finalize(prep, stats, norm)
        ctx.saved = (prep, out["lse"], out["target_prob"], norm)
        ctx.group, ctx.backend = group, backend
        ctx.in_dtypes = (x.dtype, w_shard.dtype)
        ctx.extra = dict(predicted_tokens=out["predicted_tokens"], z_loss=out["scalars"][1])
        return out["loss_rows"] if kw["reduction"] == "none" else out["scalars"][0].clone()

    @staticmethod
    def backward(ctx, grad_output):
        if ctx.stored is not None:
            gx, gw = ctx.stored
            ctx.stored = None
            dev = (gx if gx is not None else gw).device
            go = grad_output.detach().to(device=dev, dtype=torch.float32).reshape(1)
            gx = _op.scale_gradient_(gx, go)
            gw = _op.scale_gradient_(gw, go)
            h = ctx.hidden
            gx = None if gx is None else gx[:, :h].to(ctx.in_dtypes[0])
            gw = None if gw is None else gw[:, :h].to(ctx.in_dtypes[1])
            return gx, gw, None, None, None, None, None, None
        prep, lse, prob, norm = ctx.saved
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        # partial grad_input in fp32 so that the cross-rank sum is formed before the single rounding
        gx, gw = ctx.backend.backward(prep, lse, prob, norm, grad_output, need_x, need_w, grad_dtype=torch.float32)
        if need_x and _world(ctx.group) > 1:
            with _timed("all_reduce grad_input (fp32 partials)"):
                dist.all_reduce(gx, group=ctx.group)
        h = prep.hidden
        gx = None if gx is None else gx[:, :h].to(ctx.in_dtypes[0])
        gw = None if gw is None else gw[:, :h].to(ctx.in_dtypes[1])
        return gx, gw, None, None, None, None, None, None


def _kwargs(ignore_index, lse_square_scale, label_smoothing, reduction, softcap, ce_weight=None):
    assert reduction in ("mean", "sum", "none"), f"reduction must be 'mean' or 'sum' or 'none'. Got: {reduction}"
    return dict(ignore_index=ignore_index, lse_square_scale=lse_square_scale, label_smoothing=label_smoothing,
                reduction=reduction, softcap=softcap, ce_weight=ce_weight)


def token_sharded_fused_linear_cross_entropy(input, weight, target, ignore_index=-100, lse_square_scale=0.0,
                                             label_smoothing=0.0, reduction="mean", softcap=None, ce_weight=None,
                                             group=None, overlap_grad_weight=False, backend=None):
    """FLCE where each rank passes its own rows of ``input`` / ``target`` and the full ``weight``.

    Returns the loss over the *global* batch (identical on every rank; per-row for ``reduction="none"``).
    ``weight.grad`` receives the sum over ranks; ``input.grad`` is local.

    With mean / sum reduction and 16-bit operands the gradients are formed in forward and ``weight.grad`` is all-reduced
    right after the sweep (or, with ``OVERLAP_GRAD_WEIGHT``, beside the last grad_input GEMM: see the module docstring);
    a repeated backward of the same graph is not supported there.  ``overlap_grad_weight`` concerns the two-sweep path only (``reduction="none"``, fp32):
    True all-reduces each finished vocabulary slab of ``weight.grad`` on a side stream while the next slabs are
    computed.  It is off by default: those persistent GEMM kernels fill every SM, so a collective kernel that takes a
    few SMs mid-way delays whole launches (measured on 2 GPUs: 7 ms per step lost)."""
    kw = _kwargs(ignore_index, lse_square_scale, label_smoothing, reduction, softcap, ce_weight)
    kw["recording"] = torch.is_grad_enabled()
    return _TokenSharded.apply(input, weight, target, group, backend or CudaBackend(), overlap_grad_weight, kw)


def vocab_sharded_fused_linear_cross_entropy(input, weight_shard, target, vocab_start, vocab_total, ignore_index=-100,
                                             lse_square_scale=0.0, label_smoothing=0.0, reduction="mean", softcap=None,
                                             group=None, backend=None):
    """FLCE where each rank passes rows ``[vocab_start, vocab_start + V_r)`` of the weight and the full, replicated
    ``input`` / ``target`` (global class ids).  Shards must be passed in rank order of increasing ``vocab_start``.

    Returns the loss of the full problem on every rank; ``weight_shard.grad`` is local, ``input.grad`` is the sum over
    ranks (all-reduced)."""
    kw = _kwargs(ignore_index, lse_square_scale, label_smoothing, reduction, softcap)
    kw["recording"] = torch.is_grad_enabled()
    return _VocabSharded.apply(input, weight_shard, target, int(vocab_start), int(vocab_total), group,
                               backend or CudaBackend(), kw)
