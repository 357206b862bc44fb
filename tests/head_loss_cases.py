"""Shared bodies of the fused linear JSD and fused linear scaled cross-entropy tests: the same cases run on a B200
(tests/test_head_losses_gpu.py) and, with the library's SIMT kernels emulated on the host and the tensor-core
GEMM entry point replaced by torch arithmetic, on CPU tensors (tests/test_head_losses_emulation_cpu.py).

Tolerances follow the reference's tests (test/transformers/test_fused_linear_jsd.py: fp32 atol 1e-5 / rtol 5e-4, bf16
atol 5e-3 / rtol 5e-2 ... ; test_fused_linear_scaled_cross_entropy.py: fp32 6e-5 / 6e-5, bf16 8e-2 / 5e-2), tightened
where the fp64 oracle on the same rounded inputs allows it."""

import contextlib

import numpy as np
import torch

from flce_cases import assert_close
from golden_util import load_golden
from oracle.distill_oracle import fused_linear_jsd_oracle, fused_linear_scaled_ce_oracle


def _tols(dtype, vocab=0):
    # (loss atol scale, loss rtol, grad atol relative to max|g|, grad rtol)
    if dtype == torch.float32:
        # fp32 operands reach the tensor cores as bf16 term splits.  The logits carry six term products (2^-24); the two
        # projections carry dz0.w0 + dz0.w1 + dz1.w0, i.e. every product is good to about 2^-16 of its magnitude.  A
        # grad_input element sums V such products with cancellation, so its error grows with the vocabulary: 2e-5 of
        # the largest gradient entry holds up to V = 32k, 5e-4 beyond (measured 2e-4 at V = 128256).  Both are inside the
        # reference's own fp32 bar, atol 1e-5 absolute / rtol 5e-4 (test/transformers/test_fused_linear_jsd.py:94).
        return 2e-5, 2e-5, (2e-5 if vocab <= 32768 else 5e-4), 5e-4
    if dtype == torch.float16 and vocab > 100000:
        # the logit gradients of a mean over a few hundred tokens at V = 128k are about 3e-8, at fp16's smallest
        # subnormal (6e-8): an element of the 16-bit slab is 0 or one step, and a last-bit difference between the
        # kernel's approximate exp2 and the oracle's exp flips it.  The sums over V (grad_input) and over the tokens
        # (grad_weight) average the flips out to 2 - 4 % of the largest gradient entry (measured; the reference stores
        # its chunk gradients in fp16 as well).
        return 1e-2, 1e-2, 6e-2, 5e-2
    return 1e-2, 1e-2, 1e-2, 5e-2


# ---------------------------------------------------------------- fused linear JSD
def run_jsd(device, xs, ws, xt, wt, labels=None, grad_output=None, functional=False, **kw):
    import liger_kernel_b200 as lk

    xs_d = xs.to(device).clone().requires_grad_(True)
    ws_d = ws.to(device).clone().requires_grad_(True)
    args = (xs_d, ws_d, xt.to(device), wt.to(device), None if labels is None else labels.to(device))
    if functional:
        loss = lk.liger_fused_linear_jsd(*args, kw.get("jsd_beta", 0.5), kw.get("ignore_index", -100), kw.get("temperature", 1.0))
    else:
        loss = lk.LigerFusedLinearJSD(**kw)(*args)
    if grad_output is None:
        loss.backward()
    else:
        (loss * grad_output).backward()
    return dict(loss=loss.detach().float().cpu(), grad_input=xs_d.grad.float().cpu(), grad_weight=ws_d.grad.float().cpu(),
                grad_dtypes=(xs_d.grad.dtype, ws_d.grad.dtype), loss_dtype=loss.dtype)


def check_jsd(res, ora, dtype):
    l_atol, l_rtol, g_atol, g_rtol = _tols(dtype, ora.grad_weight.shape[0])
    assert res["loss_dtype"] == torch.float32 and res["grad_dtypes"] == (dtype, dtype)
    assert_close(res["loss"], ora.loss.float(), l_atol * max(1.0, float(ora.loss.abs())), l_rtol, "loss")
    for key, want in (("grad_input", ora.grad_input), ("grad_weight", ora.grad_weight)):
        assert_close(res[key], want.float(), g_atol * max(float(want.abs().max()), 1e-30), g_rtol, key)


def jsd_inputs(N, Hs, Ht, V, dtype, label_fraction=None, ignore_index=-100, seed=0):
    g = torch.Generator().manual_seed(seed)
    xs = torch.randn(N, Hs, generator=g).to(dtype)
    ws = (torch.randn(V, Hs, generator=g) * 0.3).to(dtype)
    xt = torch.randn(N, Ht, generator=g).to(dtype)
    wt = (torch.randn(V, Ht, generator=g) * 0.3).to(dtype)
    labels = None
    if label_fraction is not None:
        labels = torch.randint(0, V, (N,), generator=g)
        if ignore_index >= 0:
            labels[labels == ignore_index] = (ignore_index + 1) % V
        labels[torch.rand(N, generator=g) < label_fraction] = ignore_index
    return xs, ws, xt, wt, labels


def case_jsd_correctness(device, N, Hs, Ht, V, dtype, beta, temperature, label_fraction, ignore_index=-100, grad_output=None,
                         functional=False):
    xs, ws, xt, wt, labels = jsd_inputs(N, Hs, Ht, V, dtype, label_fraction, ignore_index, seed=N + V)
    kw = dict(jsd_beta=beta, ignore_index=ignore_index, temperature=temperature)
    res = run_jsd(device, xs, ws, xt, wt, labels, grad_output=grad_output, functional=functional, **kw)
    low = None if dtype == torch.float32 else dtype
    ora = fused_linear_jsd_oracle(xs, ws, xt, wt, labels, grad_output=1.0 if grad_output is None else grad_output,
                                  round_logits_to=low, round_dlogits_to=low, **kw)
    check_jsd(res, ora, dtype)
    if labels is not None:
        ignored = labels == ignore_index
        if bool(ignored.any()):
            assert float(res["grad_input"][ignored].abs().max()) == 0.0          # exact zeros on tokens that do not count


def case_jsd_golden(device, name):
    rec, meta = load_golden(name)
    dtype = getattr(torch, meta.get("dtype", "float32"))
    t = {k: torch.from_numpy(rec[k]).to(dtype) for k in ("student_input", "student_weight", "teacher_input", "teacher_weight")}
    labels = torch.from_numpy(rec["labels"]) if "labels" in rec else None
    kw = dict(jsd_beta=meta.get("beta", 0.5), ignore_index=meta["ignore_index"], temperature=meta.get("temperature", 1.0))
    res = run_jsd(device, t["student_input"], t["student_weight"], t["teacher_input"], t["teacher_weight"], labels,
                  grad_output=meta.get("grad_output"), **kw)
    l_atol, l_rtol, g_atol, g_rtol = _tols(dtype)
    assert_close(res["loss"], torch.from_numpy(rec["ref_loss"]), l_atol * max(1.0, float(np.abs(rec["ref_loss"]))), l_rtol,
                 "loss vs reference")
    for key in ("grad_input", "grad_weight"):
        want = torch.from_numpy(rec["ref_" + key])
        assert_close(res[key], want, g_atol * float(want.abs().max()), g_rtol, key + " vs reference")


def case_jsd_multichunk_equals_single_chunk(device, dtype=torch.bfloat16):
    """A slab budget that forces several token chunks (ragged tail included) changes nothing but the summation order of
    grad_weight."""
    import liger_kernel_b200.ops._chunked as ck

    xs, ws, xt, wt, labels = jsd_inputs(530, 24, 40, 131, dtype, 0.2, seed=5)
    kw = dict(jsd_beta=0.3, temperature=1.5)
    one = run_jsd(device, xs, ws, xt, wt, labels, **kw)
    before = ck.SLAB_BUDGET_BYTES
    ck.SLAB_BUDGET_BYTES = 256 * 2 * ck.slab_pitch(131) * (8 if dtype == torch.float32 else 2)      # 256 rows per chunk
    try:
        many = run_jsd(device, xs, ws, xt, wt, labels, **kw)
    finally:
        ck.SLAB_BUDGET_BYTES = before
    assert torch.equal(one["grad_input"], many["grad_input"])                    # rows are independent of the chunking
    np.testing.assert_allclose(one["loss"].numpy(), many["loss"].numpy(), rtol=1e-6)
    gmax = float(one["grad_weight"].abs().max())
    assert_close(many["grad_weight"], one["grad_weight"], (1e-2 if dtype != torch.float32 else 1e-6) * gmax, 1e-2, "grad_weight")


def case_jsd_all_ignored(device):
    """Every label ignored (the reference's test_correctness_all_ignored): zero loss, zero gradients, nothing undefined."""
    xs, ws, xt, wt, _ = jsd_inputs(48, 16, 32, 131, torch.bfloat16, seed=4)
    labels = torch.full((48,), 2)
    res = run_jsd(device, xs, ws, xt, wt, labels, jsd_beta=0.1, ignore_index=2, temperature=2.0)
    assert float(res["loss"]) == 0.0 and float(res["grad_input"].abs().max()) == 0.0 and float(res["grad_weight"].abs().max()) == 0.0


def case_jsd_weight_without_grad_and_second_backward(device):
    import liger_kernel_b200 as lk
    import pytest

    xs, ws, xt, wt, _ = jsd_inputs(40, 16, 16, 67, torch.bfloat16, seed=9)
    x = xs.to(device).requires_grad_(True)
    loss = lk.LigerFusedLinearJSD()(x, ws.to(device), xt.to(device), wt.to(device), None)
    loss.backward(retain_graph=True)
    assert x.grad is not None and x.grad.shape == (40, 16)
    with pytest.raises(RuntimeError, match="already handed off"):
        loss.backward()


# ---------------------------------------------------------------- fused linear scaled cross-entropy
@contextlib.contextmanager
def sce_mode(mode):
    """Run the operator in its "fused" (epilogues on the two sweeps) or "chunked" (token chunks over a logits slab) form."""
    import liger_kernel_b200.ops.fused_linear_scaled_cross_entropy as mod

    before = mod.MODE
    mod.MODE = mode
    try:
        yield
    finally:
        mod.MODE = before


def run_sce(device, x, w, t, temperature, g_nll=None, g_ent=None, ignore_index=-100, return_entropy=True):
    import liger_kernel_b200 as lk

    xd = x.to(device).clone().requires_grad_(True)
    wd = w.to(device).clone().requires_grad_(True)
    out = lk.LigerFusedLinearScaledCrossEntropyFunction.apply(xd, wd, t.to(device), temperature, ignore_index, 1, return_entropy)
    nll, entropy = out if return_entropy else (out, None)
    total = 0
    if g_nll is not None:
        total = total + (nll * g_nll.to(device)).sum()
    if g_ent is not None:
        total = total + (entropy.float() * g_ent.to(device)).sum()
    if g_nll is not None or g_ent is not None:
        total.backward()
    return dict(nll=nll.detach().float().cpu(), entropy=None if entropy is None else entropy.detach().float().cpu(),
                nll_dtype=nll.dtype, entropy_dtype=None if entropy is None else entropy.dtype,
                grad_input=None if xd.grad is None else xd.grad.float().cpu(),
                grad_weight=None if wd.grad is None else wd.grad.float().cpu())


def check_sce(res, ora, dtype, have_grads=True):
    l_atol, l_rtol, g_atol, g_rtol = _tols(dtype, ora.grad_weight.shape[0] if have_grads else 0)
    assert res["nll_dtype"] == torch.float32
    assert_close(res["nll"], ora.nll.float(), l_atol * 4, l_rtol, "nll")
    if res["entropy"] is not None:
        assert res["entropy_dtype"] == dtype
        e_atol = l_atol * 4 if dtype == torch.float32 else 4e-2          # the entropy is returned in the operands' dtype
        assert_close(res["entropy"], ora.entropy.float(), e_atol, l_rtol, "entropy")
    if have_grads:
        for key, want in (("grad_input", ora.grad_input), ("grad_weight", ora.grad_weight)):
            assert_close(res[key], want.float(), g_atol * max(float(want.abs().max()), 1e-30), g_rtol, key)


def sce_inputs(N, H, V, dtype, ignored=0.1, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(N, H, generator=g) * 0.5).to(dtype)
    w = (torch.randn(V, H, generator=g) / H ** 0.5 * 2).to(dtype)
    t = torch.randint(0, V, (N,), generator=g)
    t[torch.rand(N, generator=g) < ignored] = -100
    return x, w, t, torch.randn(N, generator=g), torch.randn(N, generator=g)


def case_sce_correctness(device, N, H, V, dtype, temperature, grads="both", mode="fused"):
    x, w, t, g_nll, g_ent = sce_inputs(N, H, V, dtype, seed=N + V)
    g_nll = g_nll if grads in ("both", "nll") else None
    g_ent = g_ent if grads in ("both", "entropy") else None
    with sce_mode(mode):
        res = run_sce(device, x, w, t, temperature, g_nll, g_ent)
    low = None if dtype == torch.float32 else dtype
    ora = fused_linear_scaled_ce_oracle(x, w, t, temperature, -100, g_nll, g_ent, round_logits_to=low, round_dlogits_to=low)
    check_sce(res, ora, dtype)
    ignored = t == -100
    if bool(ignored.any()):
        assert float(res["nll"][ignored].abs().max()) == 0.0 and float(res["entropy"][ignored].abs().max()) == 0.0
        assert float(res["grad_input"][ignored].abs().max()) == 0.0


def case_sce_golden(device, name, mode="fused"):
    rec, meta = load_golden(name)
    dtype = getattr(torch, meta.get("dtype", "float32"))
    x, w, t = torch.from_numpy(rec["x"]).to(dtype), torch.from_numpy(rec["w"]).to(dtype), torch.from_numpy(rec["target"])
    g_nll = torch.from_numpy(rec["grad_nll"]) if meta["grads"] in ("both", "nll") else None
    g_ent = torch.from_numpy(rec["grad_entropy"]) if meta["grads"] in ("both", "entropy") else None
    with sce_mode(mode):
        res = run_sce(device, x, w, t, meta["temperature"], g_nll, g_ent)
    l_atol, l_rtol, g_atol, g_rtol = _tols(dtype)
    low = dtype != torch.float32
    assert_close(res["nll"], torch.from_numpy(rec["ref_nll"]), 4e-2 if low else 8e-5, l_rtol, "nll vs reference")
    assert_close(res["entropy"], torch.from_numpy(rec["ref_entropy"]), 8e-2 if low else 8e-5, l_rtol, "entropy vs reference")
    for key in ("grad_input", "grad_weight"):
        want = torch.from_numpy(rec["ref_" + key])
        assert_close(res[key], want, (2e-2 if low else g_atol) * float(want.abs().max()), g_rtol, key + " vs reference")


def case_sce_nll_only_output_and_no_grad(device):
    """return_entropy=False gives one tensor; under no_grad nothing is kept for backward."""
    import liger_kernel_b200 as lk

    x, w, t, _, _ = sce_inputs(33, 24, 97, torch.float16, seed=3)
    with torch.no_grad():
        nll = lk.LigerFusedLinearScaledCrossEntropyFunction.apply(x.to(device), w.to(device), t.to(device), 0.9)
    assert torch.is_tensor(nll) and nll.shape == (33,) and nll.dtype == torch.float32
    ora = fused_linear_scaled_ce_oracle(x, w, t, 0.9, round_logits_to=torch.float16)
    assert_close(nll.cpu(), ora.nll.float(), 2e-2, 1e-2, "nll")


def case_sce_argument_errors(device):
    import liger_kernel_b200 as lk
    import pytest

    x, w, t, _, _ = sce_inputs(8, 16, 32, torch.bfloat16)
    x, w, t = x.to(device), w.to(device), t.to(device)
    f = lk.LigerFusedLinearScaledCrossEntropyFunction.apply
    with pytest.raises(ValueError, match="temperature must be finite and > 0"):
        f(x, w, t, 0.0)
    with pytest.raises(TypeError, match="temperature must be a real number"):
        f(x, w, t, "1")
    with pytest.raises(TypeError, match="m_tiles_per_cluster must be an int"):
        f(x, w, t, 1.0, -100, 1.5)
    with pytest.raises(ValueError, match="m_tiles_per_cluster must be >= 1"):
        f(x, w, t, 1.0, -100, 0)
    with pytest.raises(TypeError, match="return_entropy must be a bool"):
        f(x, w, t, 1.0, -100, 1, 1)
    with pytest.raises(TypeError, match="target must be an int64 tensor"):
        f(x, w, t.int(), 1.0)
    with pytest.raises(ValueError, match="shapes are incompatible"):
        f(x, w[:, :8], t, 1.0)
    with pytest.raises(TypeError, match="same floating-point dtype"):
        f(x, w.float(), t, 1.0)
