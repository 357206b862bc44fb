"""Parity of the CUDA path (through the public API and the C ABI below it) with the CPU oracle and with
the golden vectors of the reference.  Case grid follows the reference's
test/transformers/test_fused_linear_cross_entropy.py (shapes (8,128,1024,4096) and (4,47,31,123), feature
rows, bias on/off, mean/sum/none) and test/cutedsl/test_fused_linear_cross_entropy.py (ragged row counts,
odd vocabulary, all-ignored rows, upstream gradient != 1, repeated backward).

Tolerances: loss 1e-4 relative, per-row lse 1e-5 (relative to max(1,|lse|)) against fp64 math on the same
16-bit inputs; gradients atol 1e-2 / rtol 5e-2 of the bf16 bar, tightened by the gradient scale where noted;
ignored rows and integer outputs exact.
"""

import ctypes as C

import numpy as np
import pytest
import torch

from flce_cases import assert_close, make_inputs, oracle_for, run_cuda
from golden_util import golden_grad_output, golden_kwargs, golden_names, load_golden

pytestmark = pytest.mark.gpu


def _check(res, ora, dtype, reduction, n_rows):
    scale = max(1.0, float(ora.loss.abs().max()))
    assert_close(res["loss"], ora.loss.float(), 1e-4 * scale, 1e-4, "loss")
    assert_close(res["z_loss"].float(), ora.z_loss.float(), 2e-2 * max(1e-3, float(ora.z_loss.abs().max())), 1e-2, "z_loss")
    assert torch.equal(res["predicted_tokens"] == -1, ora.predicted_tokens == -1)
    # arg-max of the row: exact except where the two best logits are closer than the 16-bit operands' fp32 accumulation
    # order can resolve (a handful of rows at most), and the accuracy built from it
    live = ora.predicted_tokens != -1
    if bool(live.any()):
        differ = int((res["predicted_tokens"][live] != ora.predicted_tokens[live]).sum())
        assert differ <= max(1, int(0.005 * int(live.sum()))), f"{differ} of {int(live.sum())} predicted tokens differ"
        if reduction != "none" and "token_accuracy" in res:
            assert abs(float(res["token_accuracy"]) - float(ora.token_accuracy)) <= 0.005 + 1.0 / int(live.sum())
    # gradient magnitude: mean divides by the row count, 16-bit storage rounds relative to the value
    # the bar is atol 1e-2 / rtol 5e-2; the absolute part is tightened to one bf16 ulp-ish (2^-7) of each
    # tensor's largest entry so that small-magnitude gradients (mean reduction) are still checked.  Un-normalised
    # reductions (sum, none) give gradients of order 1 to 10, where one 16-bit ulp of the largest entry already exceeds
    # 1e-2 and an element that is a small difference of large terms carries that much absolute error: there the bar
    # stays relative to the largest entry (the reference's own bar for 16-bit sum is atol 5 / rtol 50,
    # test/transformers/test_fused_linear_cross_entropy.py:120).
    for key, want in (("grad_input", ora.grad_input), ("grad_weight", ora.grad_weight), ("grad_bias", ora.grad_bias)):
        if res.get(key) is None:
            continue
        atol = 8e-3 * max(float(want.abs().max()), 1e-30)
        if reduction == "mean":
            atol = min(1e-2, atol)
        assert_close(res[key].float(), want.float(), atol, 5e-2, key)


FEATURES = [
    dict(),
    dict(label_smoothing=0.1),
    dict(lse_square_scale=1e-4),
    dict(softcap=30.0),
    dict(label_smoothing=0.1, ignore_index=42, lse_square_scale=1e-4, softcap=30.0),
]


@pytest.mark.parametrize("B,T,H,V", [(8, 128, 1024, 4096), (4, 47, 31, 123)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("reduction", ["mean", "sum"])
@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("feat", FEATURES)
def test_correctness(B, T, H, V, dtype, reduction, bias, feat):
    x, w, t, b, _ = make_inputs(B * T, H, V, dtype, seed=B * T + V, bias=bias, ignore_index=feat.get("ignore_index", -100))
    kw = dict(reduction=reduction, **feat)
    res = run_cuda(x, w, t, bias=b, **kw)
    ora = oracle_for(x, w, t, bias=b, **kw)
    _check(res, ora, dtype, reduction, B * T)


@pytest.mark.parametrize("N", [129, 640, 1269])
@pytest.mark.parametrize("H,V", [(512, 4096), (127, 513), (2048, 32000)])
def test_ragged_shapes_and_lse(N, H, V):
    """Row tails, odd vocabulary (padding columns must never enter max / sum / arg-max) and per-row lse."""
    from liger_kernel_b200.ops.fused_linear_cross_entropy import _Prepared, flce_forward_device

    x, w, t, _, _ = make_inputs(N, H, V, torch.bfloat16, seed=N + V, wscale=0.05)
    ora = oracle_for(x, w, t)
    prep = _Prepared(x.cuda(), w.cuda(), t.cuda(), None, None, -100, 0.0, 0.0, "mean", None, False)
    out, norm, _ = flce_forward_device(prep)
    lse = out["lse"].cpu().double()
    valid = t != -100
    want = ora.lse.double()
    err = ((lse - want).abs() / want.abs().clamp(min=1.0))[valid]
    assert float(err.max()) <= 1e-5, f"lse error {float(err.max()):.3e}"
    assert int(norm[0].item()) == int(valid.sum())
    assert torch.equal(out["predicted_tokens"].cpu(), ora.predicted_tokens)
    assert_close(out["scalars"][0].cpu(), ora.loss.float(), 0, 1e-4, "loss")
    res = run_cuda(x, w, t)
    _check(res, ora, torch.bfloat16, "mean", N)


def test_all_rows_ignored_exact_zero():
    x, w, t, _, _ = make_inputs(256, 128, 1000, torch.bfloat16, seed=3, ignore_frac=1.1)
    res = run_cuda(x, w, t)
    assert float(res["loss"]) == 0.0
    assert float(res["grad_input"].abs().max()) == 0.0 and float(res["grad_weight"].abs().max()) == 0.0
    assert torch.all(res["predicted_tokens"] == -1)


def test_ignored_rows_have_exact_zero_gradient():
    x, w, t, _, _ = make_inputs(300, 256, 777, torch.bfloat16, seed=4, ignore_frac=0.4)
    res = run_cuda(x, w, t, lse_square_scale=1e-3, label_smoothing=0.1)
    assert float(res["grad_input"][t == -100].abs().max()) == 0.0


def test_targets_at_vocab_edges():
    x, w, t, _, _ = make_inputs(260, 64, 1030, torch.bfloat16, seed=5, ignore_frac=0.0)
    t[::2] = 0
    t[1::2] = 1029
    res = run_cuda(x, w, t)
    _check(res, oracle_for(x, w, t), torch.bfloat16, "mean", 260)


@pytest.mark.parametrize("go", [2.0, 0.5])
def test_grad_output_scalar(go):
    x, w, t, _, _ = make_inputs(200, 96, 500, torch.bfloat16, seed=6)
    res = run_cuda(x, w, t, grad_output=go)
    ora = oracle_for(x, w, t, grad_output=go)
    _check(res, ora, torch.bfloat16, "mean", 200)


def test_reduction_none_per_token_grad():
    x, w, t, _, _ = make_inputs(200, 96, 500, torch.bfloat16, seed=7)
    go = torch.rand(200) + 0.5
    res = run_cuda(x, w, t, reduction="none", grad_output=go)
    ora = oracle_for(x, w, t, reduction="none", grad_output=go)
    assert_close(res["loss"], ora.loss.float(), 1e-4, 1e-4, "loss rows")
    assert_close(res["grad_input"].float(), ora.grad_input.float(), 1e-2, 5e-2, "grad_input")
    assert_close(res["grad_weight"].float(), ora.grad_weight.float(), 1e-2, 5e-2, "grad_weight")


def test_token_scaling_and_class_weights():
    x, w, t, _, cw = make_inputs(200, 96, 500, torch.bfloat16, seed=8, ce_weight=True)
    for kw in (dict(use_token_scaling=True), dict(label_smoothing=0.1), dict()):
        use_cw = None if kw.get("use_token_scaling") else cw
        res = run_cuda(x, w, t, ce_weight=use_cw, **kw)
        ora = oracle_for(x, w, t, ce_weight=use_cw, **kw)
        _check(res, ora, torch.bfloat16, "mean", 200)
    # both together, in every mode: class weights scale the row's loss, token scaling multiplies it by the (detached)
    # probability of the target
    import liger_kernel_b200.ops.fused_linear_cross_entropy as mod
    for mode in ("auto", "recompute"):
        old, mod.MODE = mod.MODE, mode
        try:
            for kw in (dict(use_token_scaling=True), dict(use_token_scaling=True, label_smoothing=0.1, lse_square_scale=1e-4)):
                res = run_cuda(x, w, t, ce_weight=cw, **kw)
                _check(res, oracle_for(x, w, t, ce_weight=cw, **kw), torch.bfloat16, "mean", 200)
        finally:
            mod.MODE = old


def test_repeated_backward_doubles_exactly(monkeypatch):
    """Two-sweep mode: backward is a pure function of what forward saved, so a second call adds the same bits again.
    (In the default mode the first backward hands off gradients formed in forward and a repeat recomputes them:
    test_single_sweep_all_ignored_and_repeated_backward.)"""
    import liger_kernel_b200.ops.fused_linear_cross_entropy as mod
    from liger_kernel_b200.ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction as Fn

    monkeypatch.setattr(mod, "MODE", "recompute")
    x, w, t, _, _ = make_inputs(200, 96, 500, torch.bfloat16, seed=9)
    xd, wd = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    loss = Fn.apply(xd, wd, t.cuda())[0]
    loss.backward(retain_graph=True)
    g1x, g1w = xd.grad.clone(), wd.grad.clone()
    loss.backward()
    assert torch.equal(xd.grad, 2 * g1x) and torch.equal(wd.grad, 2 * g1w)


def test_run_to_run_bitwise_determinism():
    x, w, t, _, _ = make_inputs(700, 256, 3000, torch.bfloat16, seed=10)
    a = run_cuda(x, w, t, label_smoothing=0.1)
    b = run_cuda(x, w, t, label_smoothing=0.1)
    for k in ("loss", "grad_input", "grad_weight"):
        assert torch.equal(a[k], b[k]), k


def test_multi_slab_backward_matches_single_slab(monkeypatch):
    """Two-sweep mode: a small slab budget forces several vocabulary slabs: dX is accumulated across them in fp32."""
    import liger_kernel_b200.ops.fused_linear_cross_entropy as mod

    monkeypatch.setattr(mod, "MODE", "recompute")
    x, w, t, b, _ = make_inputs(384, 128, 2000, torch.bfloat16, seed=11, bias=True)
    one = run_cuda(x, w, t, bias=b)
    old = mod.SLAB_BUDGET_BYTES
    mod.SLAB_BUDGET_BYTES = 384 * 2 * 512  # 512 columns per slab -> 4 slabs
    try:
        many = run_cuda(x, w, t, bias=b)
    finally:
        mod.SLAB_BUDGET_BYTES = old
    assert torch.equal(one["grad_weight"], many["grad_weight"])
    assert torch.equal(one["grad_bias"], many["grad_bias"])
    assert_close(many["grad_input"].float(), one["grad_input"].float(), 1e-5, 2e-2, "grad_input")
    _check(many, oracle_for(x, w, t, bias=b), torch.bfloat16, "mean", 384)


def test_cta_pair_matches_single_cta():
    from liger_kernel_b200 import _lib

    x, w, t, _, _ = make_inputs(700, 256, 3000, torch.bfloat16, seed=12)
    a = run_cuda(x, w, t)
    _lib.set_option("cta_pair", 0)
    try:
        b = run_cuda(x, w, t)
    finally:
        _lib.set_option("cta_pair", 1)
    assert_close(b["loss"], a["loss"], 0, 1e-6, "loss")
    assert_close(b["grad_weight"].float(), a["grad_weight"].float(), 1e-6, 1e-2, "grad_weight")
    _check(b, oracle_for(x, w, t), torch.bfloat16, "mean", 700)


@pytest.mark.parametrize("name", golden_names())
def test_against_reference_golden(name):
    rec, meta = load_golden(name)
    x, w, t = torch.from_numpy(rec["x"]).bfloat16(), torch.from_numpy(rec["w"]).bfloat16(), torch.from_numpy(rec["target"])
    kw = golden_kwargs(rec, meta)
    bias, cw = kw.pop("bias"), kw.pop("ce_weight")
    bias = None if bias is None else bias.bfloat16()
    go = golden_grad_output(rec, meta)
    res = run_cuda(x, w, t, bias=bias, ce_weight=cw, grad_output=go, **kw)
    # the golden outputs were produced from the fp32 inputs: bf16 rounding of x and w bounds the agreement
    scale = max(1.0, float(np.abs(rec["ref_loss"]).max()))
    tol = 5e-2 if name == "token_scaling" else 2e-2
    assert_close(res["loss"], torch.from_numpy(rec["ref_loss"]), tol * scale, tol, "loss vs reference")
    gs = max(float(np.abs(rec["ref_grad_weight"]).max()), 1e-6)
    assert_close(res["grad_weight"].float(), torch.from_numpy(rec["ref_grad_weight"]), 5e-2 * gs, 1e-1, "grad_weight vs reference")
    gs = max(float(np.abs(rec["ref_grad_input"]).max()), 1e-6)
    assert_close(res["grad_input"].float(), torch.from_numpy(rec["ref_grad_input"]), 5e-2 * gs, 1e-1, "grad_input vs reference")
    # and tightly against the oracle on the same rounded inputs
    ora = oracle_for(x, w, t, bias=bias, ce_weight=cw, grad_output=go, **kw)
    _check(res, ora, torch.bfloat16, kw["reduction"], x.shape[0])


def test_error_paths():
    from liger_kernel_b200 import _lib
    from liger_kernel_b200.ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction as Fn

    x = torch.randn(16, 64, dtype=torch.bfloat16)
    w = torch.randn(100, 64, dtype=torch.bfloat16)
    t = torch.randint(0, 100, (16,))
    with pytest.raises(RuntimeError):  # CPU tensors: no fallback
        Fn.apply(x, w, t)
    with pytest.raises(ValueError):
        Fn.apply(x.cuda(), w.cuda(), t.cuda(), None, None, -100, 0.0, 0.0, "median")
    with pytest.raises(TypeError):
        Fn.apply(x.cuda().half(), w.cuda(), t.cuda())
    rc = _lib.lib.flce_b200_gemm(None, None, None, 1, 8, 8, 8, 8, 8, 0, 2, 0, 0, 0, None)
    assert rc == 1 and b"NULL" in _lib.lib.flce_b200_last_error()
    loss = Fn.apply(x.cuda(), w.cuda(), t.cuda())[0]
    with pytest.raises(RuntimeError, match="does not require grad"):
        loss.backward()


def test_full_size_properties():
    """Llama-3-8B head size (N=32768, H=4096, V=128256): size-independent properties plus sampled rows and
    sampled vocabulary rows against fp64 math on the CPU."""
    from liger_kernel_b200.ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction as Fn

    if torch.cuda.get_device_properties(0).total_memory < 40e9:
        pytest.skip("needs ~10 GB of device memory")
    N, H, V = 32768, 4096, 128256
    g = torch.Generator(device="cuda").manual_seed(2024)
    x = torch.randn(N, H, generator=g, device="cuda").bfloat16()
    w = (torch.randn(V, H, generator=g, device="cuda") * 0.02).bfloat16()
    t = torch.randint(0, V, (N,), generator=g, device="cuda")
    t[torch.rand(N, generator=g, device="cuda") < 0.05] = -100
    xd, wd = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    loss = Fn.apply(xd, wd, t)[0]
    loss.backward()
    rows = Fn.apply(x, w, t, None, None, -100, 0.0, 0.0, "none")[0]
    n_valid = int((t != -100).sum())
    # mean == sum of per-row losses / count
    assert abs(float(rows.double().sum()) / n_valid - float(loss.detach())) <= 1e-5 * abs(float(loss.detach()))
    # ignored rows: exact zeros
    assert float(xd.grad[t == -100].abs().max()) == 0.0 and float(rows[t == -100].abs().max()) == 0.0
    # linearity in the upstream gradient (power of two: bit exact)
    x2, w2 = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    Fn.apply(x2, w2, t)[0].backward(torch.tensor(2.0, device="cuda"))
    assert torch.equal(x2.grad, 2 * xd.grad) and torch.equal(w2.grad, 2 * wd.grad)
    del x2, w2
    # sampled token rows against fp64
    from liger_kernel_b200.ops.fused_linear_cross_entropy import _Prepared, flce_forward_device

    out, _, _ = flce_forward_device(_Prepared(x, w, t, None, None, -100, 0.0, 0.0, "mean", None, False))
    lse = out["lse"]
    pick = torch.arange(0, N, 509, device="cuda")[:64]
    wf = w.double()
    z = x[pick].double() @ wf.t()
    lse_ref = torch.logsumexp(z, dim=1)
    assert float(((lse[pick].double() - lse_ref).abs() / lse_ref.abs().clamp(min=1)).max()) <= 1e-5
    p = torch.exp(z - lse_ref[:, None])
    valid = (t[pick] != -100)
    onehot = torch.zeros_like(p)
    onehot[torch.arange(len(pick), device="cuda")[valid], t[pick][valid]] = 1.0
    gz = (p - onehot) * valid[:, None] / n_valid
    dx_ref = gz @ wf
    assert_close(xd.grad[pick].float().cpu(), dx_ref.float().cpu(), 8e-3 * float(dx_ref.abs().max()), 5e-2, "grad_input rows")
    # sampled vocabulary rows of grad_weight (uses the per-row lse validated above)
    vs = torch.tensor([0, 1, 4097, 65000, 128000, 128255], device="cuda")
    zc = x.double() @ wf[vs].t()                                  # [N, 6]
    pc = torch.exp(zc - lse.double()[:, None])
    hit = (t[:, None] == vs[None, :]).double()
    gc = (pc - hit) * (t != -100)[:, None] / n_valid
    dw_ref = gc.t() @ x.double()
    assert_close(wd.grad[vs].float().cpu(), dw_ref.float().cpu(), 8e-3 * float(dw_ref.abs().max()), 5e-2, "grad_weight rows")


# ---------------------------------------------------------------------------------------------------------------
# single-sweep mode (gradients formed in forward from a 16-bit copy of each token chunk's logits)
# ---------------------------------------------------------------------------------------------------------------
@pytest.fixture
def single_sweep(monkeypatch):
    import liger_kernel_b200.ops.fused_linear_cross_entropy as mod

    monkeypatch.setattr(mod, "MODE", "single_sweep")
    return mod


@pytest.fixture
def recompute(monkeypatch):
    import liger_kernel_b200.ops.fused_linear_cross_entropy as mod

    monkeypatch.setattr(mod, "MODE", "recompute")
    return mod


@pytest.mark.parametrize("B,T,H,V", [(8, 128, 1024, 4096), (4, 47, 31, 123)])
@pytest.mark.parametrize("reduction", ["mean", "sum"])
@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("feat", FEATURES)
def test_recompute_correctness(recompute, B, T, H, V, reduction, bias, feat):
    """The two-sweep mode on the grid that the default mode (gradients formed in forward) covers in test_correctness."""
    test_correctness(B, T, H, V, torch.bfloat16, reduction, bias, feat)


@pytest.mark.parametrize("B,T,H,V", [(8, 128, 1024, 4096), (4, 47, 31, 123)])
@pytest.mark.parametrize("reduction", ["mean", "sum"])
@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("feat", FEATURES)
@pytest.mark.parametrize("store", ["auto", "logits"])
def test_single_sweep_correctness(single_sweep, monkeypatch, B, T, H, V, reduction, bias, feat, store):
    """Both forms of the bounded 16-bit copy: the logits themselves, and (auto, wherever it applies: bf16, no bias
    gradient, no label smoothing under a soft-cap) their exponentials against a per-row reference point."""
    monkeypatch.setattr(single_sweep, "STORE_MODE", store)
    x, w, t, b, _ = make_inputs(B * T, H, V, torch.bfloat16, seed=B * T + V + 1, bias=bias,
                                ignore_index=feat.get("ignore_index", -100))
    kw = dict(reduction=reduction, **feat)
    res = run_cuda(x, w, t, bias=b, **kw)
    _check(res, oracle_for(x, w, t, bias=b, **kw), torch.bfloat16, reduction, B * T)


def test_exp_store_rows_far_from_their_reference_point(single_sweep):
    """Rows that miss their target by hundreds of nats cannot be expressed against the target logit: the chunk goes
    through sweep 1 a second time with the reference points on the log-sum-exp, decided on the device.  Large logits
    are also where rounded stored logits would lose the softmax (one bf16 ulp of 200 is 1): exponentials keep it."""
    g = torch.Generator().manual_seed(4)
    x = torch.randn(700, 64, generator=g).bfloat16()
    w = (torch.randn(3000, 64, generator=g) * 6).bfloat16()
    t = torch.randint(0, 3000, (700,), generator=g)
    t[:350] = (x.double() @ w.double().T)[:350].argmax(1)
    for kw in (dict(), dict(label_smoothing=0.1, lse_square_scale=1e-4), dict(softcap=30.0)):
        res = run_cuda(x, w, t, **kw)
        assert bool(torch.isfinite(res["grad_input"].float()).all()) and bool(torch.isfinite(res["grad_weight"].float()).all())
        _check(res, oracle_for(x, w, t, **kw), torch.bfloat16, "mean", 700)


def test_single_sweep_many_chunks_weights_scaling_and_upstream_gradient(single_sweep, monkeypatch):
    x, w, t, b, cw = make_inputs(1100, 96, 700, torch.bfloat16, seed=21, bias=True, ce_weight=True)
    monkeypatch.setattr(single_sweep, "CHUNK_BUDGET_BYTES", 256 * 704 * 2)      # 256-row chunks -> 5 chunks
    for kw, use_cw, go in ((dict(label_smoothing=0.1), cw, None), (dict(use_token_scaling=True), None, None),
                           (dict(lse_square_scale=1e-3), None, 2.5)):
        res = run_cuda(x, w, t, bias=b, ce_weight=use_cw, grad_output=go, **kw)
        ora = oracle_for(x, w, t, bias=b, ce_weight=use_cw, grad_output=go, **kw)
        _check(res, ora, torch.bfloat16, "mean", 1100)


def test_single_sweep_all_ignored_and_repeated_backward(single_sweep):
    from liger_kernel_b200.ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction as Fn

    x, w, t, _, _ = make_inputs(256, 128, 1000, torch.bfloat16, seed=3, ignore_frac=1.1)
    res = run_cuda(x, w, t)
    assert float(res["loss"]) == 0.0 and float(res["grad_input"].abs().max()) == 0.0 and float(res["grad_weight"].abs().max()) == 0.0
    x, w, t, _, _ = make_inputs(200, 96, 500, torch.bfloat16, seed=9)
    xd, wd = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    loss = Fn.apply(xd, wd, t.cuda())[0]
    loss.backward(retain_graph=True)          # stored gradients
    g1 = wd.grad.clone()
    loss.backward()                           # second time: recompute sweep
    assert_close((wd.grad - g1).float().cpu(), g1.float().cpu(), 8e-3 * float(g1.abs().max()), 5e-2, "second backward")
    # reduction "none" is served by the two-sweep path even in this mode
    res = run_cuda(x, w, t, reduction="none", grad_output=torch.rand(200) + 0.5)
    assert res["grad_input"].shape == (200, 96)


# ---------------------------------------------------------------------------------------------------------------
# fp32 inputs: 16-bit term splits on the same tensor-core kernels
# ---------------------------------------------------------------------------------------------------------------
def _check_fp32(res, ora, reduction, wide=False):
    scale = max(1.0, float(ora.loss.abs().max()))
    # reference bars for fp32: mean 1e-5 / 5e-4, sum 1e-3 / 5e-2 (test_fused_linear_cross_entropy.py:115-123)
    assert_close(res["loss"], ora.loss.float(), 1e-5 * scale, 2e-5, "loss")
    # The gradient projections run on two bf16 terms of dZ and of x / w (dz0.t0 + dz0.t1 + dz1.t0): each product is good
    # to about 2^-16, and a grad_input element sums V of them with cancellation.  2e-5 of the largest entry holds up to
    # V = 32k; at V = 128k the measured error is 2e-4, so the wide case uses 5e-4 (still inside the reference's bar).
    g_atol = 5e-4 if wide else 2e-5
    for key, want in (("grad_input", ora.grad_input), ("grad_weight", ora.grad_weight), ("grad_bias", ora.grad_bias)):
        if res.get(key) is None:
            continue
        atol = g_atol * max(float(want.abs().max()), 1e-30)
        assert_close(res[key].float(), want.float(), atol, 5e-4, key)


@pytest.mark.parametrize("B,T,H,V", [(8, 128, 1024, 4096), (4, 47, 31, 123)])
@pytest.mark.parametrize("reduction", ["mean", "sum"])
@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("feat", FEATURES)
def test_correctness_fp32(B, T, H, V, reduction, bias, feat):
    x, w, t, b, _ = make_inputs(B * T, H, V, torch.float32, seed=B * T + V + 2, bias=bias,
                                ignore_index=feat.get("ignore_index", -100))
    kw = dict(reduction=reduction, **feat)
    res = run_cuda(x, w, t, bias=b, **kw)
    assert res["grad_input"].dtype == torch.float32 and res["z_loss"].dtype == torch.float32
    _check_fp32(res, oracle_for(x, w, t, bias=b, **kw), reduction)


def test_config_c1_small_fp32_head():
    """Benchmark configuration 1: N=1024 (B=2, T=512), H=1024, V=32000, fp32, X~N(0,1), W~N(0,1/H), 10 % ignored, mean."""
    from liger_kernel_b200.ops.fused_linear_cross_entropy import _Prepared, flce_forward_device

    x, w, t, _, _ = make_inputs(1024, 1024, 32000, torch.float32, seed=1234 + 1, ignore_frac=0.10, wscale=1024 ** -0.5)
    ora = oracle_for(x, w, t)
    res = run_cuda(x, w, t)
    _check_fp32(res, ora, "mean")
    prep = _Prepared(x.cuda(), w.cuda(), t.cuda(), None, None, -100, 0.0, 0.0, "mean", None, False)
    out, _, _ = flce_forward_device(prep)
    valid = t != -100
    err = ((out["lse"].cpu().double() - ora.lse) .abs() / ora.lse.abs().clamp(min=1.0))[valid]
    assert float(err.max()) <= 1e-5, float(err.max())
    assert torch.equal(out["predicted_tokens"].cpu(), ora.predicted_tokens)


def test_fp32_wide_vocabulary():
    """fp32 operands at the Llama-3 vocabulary (V = 128256): the reduction over V in grad_input is 4x longer than in C1."""
    x, w, t, _, _ = make_inputs(256, 128, 128256, torch.float32, seed=77, ignore_frac=0.1)
    kw = dict(label_smoothing=0.1, lse_square_scale=1e-4)
    res = run_cuda(x, w, t, **kw)
    _check_fp32(res, oracle_for(x, w, t, **kw), "mean", wide=True)


@pytest.mark.parametrize("name", ["mean_default", "all_features", "qwen_style", "gemma_style_sum", "none_reduction", "ce_weight"])
def test_golden_fp32_inputs_against_reference_outputs(name):
    """fp32 inputs exactly as the reference saw them: outputs must agree with the reference's own to fp32 accuracy."""
    rec, meta = load_golden(name)
    x, w, t = torch.from_numpy(rec["x"]), torch.from_numpy(rec["w"]), torch.from_numpy(rec["target"])
    kw = golden_kwargs(rec, meta)
    bias, cw = kw.pop("bias"), kw.pop("ce_weight")
    go = golden_grad_output(rec, meta)
    res = run_cuda(x, w, t, bias=bias, ce_weight=cw, grad_output=go, **kw)
    scale = max(1.0, float(np.abs(rec["ref_loss"]).max()))
    assert_close(res["loss"], torch.from_numpy(rec["ref_loss"]), 2e-5 * scale, 2e-4, "loss vs reference")
    for key in ("grad_input", "grad_weight"):
        want = torch.from_numpy(rec["ref_" + key])
        assert_close(res[key].float(), want, 5e-5 * float(want.abs().max()), 1e-3, key + " vs reference")

