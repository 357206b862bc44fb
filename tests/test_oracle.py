"""The CPU oracle against the golden vectors produced by the reference itself.

Mirrors the comparisons of test/transformers/test_fused_linear_cross_entropy.py
(reference) with stored outputs instead of a live GPU run.
"""

import numpy as np
import pytest
import torch

from golden_util import golden_grad_output, golden_kwargs, golden_names, jsd_golden_names, load_golden, sce_golden_names
from oracle.distill_oracle import fused_linear_jsd_oracle, fused_linear_scaled_ce_oracle
from oracle.flce_oracle import flce_oracle, torch_linear_ce_reference


def _close(a, b, atol, rtol, what):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape, (what, a.shape, b.shape)
    err = np.abs(a - b) - (atol + rtol * np.abs(b))
    assert np.all(err <= 0), f"{what}: max excess {err.max():.3e}, max abs diff {np.abs(a-b).max():.3e}"


@pytest.mark.parametrize("name", golden_names())
def test_oracle_matches_reference_golden(name):
    rec, meta = load_golden(name)
    bf16 = meta.get("dtype") == "bfloat16"
    x, w, t = torch.from_numpy(rec["x"]), torch.from_numpy(rec["w"]), torch.from_numpy(rec["target"])
    res = flce_oracle(x, w, t, grad_output=golden_grad_output(rec, meta), **golden_kwargs(rec, meta))
    # fp32 reference kernels vs fp64 closed form; the bf16 case carries the reference's bf16 logits rounding
    atol, rtol = (2e-2, 2e-2) if bf16 else (2e-5, 2e-4)
    if name == "softcap_padded_quirk":
        # the reference soft-caps its -inf padding into -softcap (see make_golden.py); the oracle follows torch
        atol, rtol = 1e-2, 1e-2
    scale = max(1.0, float(np.abs(rec["ref_loss"]).max()))
    _close(res.loss, rec["ref_loss"], atol * scale, rtol, "loss")
    if "ref_z_loss" in rec:
        _close(res.z_loss, rec["ref_z_loss"], atol, rtol, "z_loss")
    gatol = 2e-3 if bf16 else 2e-6 * max(1.0, float(np.abs(rec["ref_grad_weight"]).max()))
    if name == "softcap_padded_quirk":
        gatol = 1e-4
    _close(res.grad_input, rec["ref_grad_input"], gatol, 5e-2 if bf16 else 1e-3, "grad_input")
    _close(res.grad_weight, rec["ref_grad_weight"], gatol, 5e-2 if bf16 else 1e-3, "grad_weight")
    if "ref_grad_bias" in rec:
        _close(res.grad_bias, rec["ref_grad_bias"], gatol, 1e-3, "grad_bias")
    if "ref_token_accuracy" in rec:
        _close(res.token_accuracy, rec["ref_token_accuracy"], 1e-6, 0, "token_accuracy")
    if "ref_predicted_tokens" in rec:
        assert np.array_equal(res.predicted_tokens.numpy(), rec["ref_predicted_tokens"])


@pytest.mark.parametrize("name", [n for n in golden_names()])
def test_oracle_matches_torch_ground_truth(name):
    rec, meta = load_golden(name)
    if "torch_loss" not in rec or meta["ign"] >= 1.0:
        pytest.skip("no torch equivalent for this case (torch gives nan when every row is ignored)")
    x, w, t = torch.from_numpy(rec["x"]), torch.from_numpy(rec["w"]), torch.from_numpy(rec["target"])
    res = flce_oracle(x, w, t, **golden_kwargs(rec, meta))
    scale = max(1.0, float(np.abs(rec["torch_loss"]).max()))
    _close(res.loss, rec["torch_loss"], 2e-5 * scale, 2e-4, "loss")
    if "torch_grad_input" in rec:
        _close(res.grad_input, rec["torch_grad_input"], 1e-5, 1e-3, "grad_input")
        _close(res.grad_weight, rec["torch_grad_weight"], 1e-5, 1e-3, "grad_weight")


def test_all_ignored_is_exact_zero():
    rec, meta = load_golden("all_ignored")
    x, w, t = torch.from_numpy(rec["x"]), torch.from_numpy(rec["w"]), torch.from_numpy(rec["target"])
    res = flce_oracle(x, w, t, **golden_kwargs(rec, meta))
    assert float(res.loss) == 0.0
    assert float(res.grad_input.abs().max()) == 0.0 and float(res.grad_weight.abs().max()) == 0.0
    assert np.all(rec["ref_grad_input"] == 0) and np.all(rec["ref_grad_weight"] == 0) and rec["ref_loss"] == 0


def test_closed_form_equals_autograd_fp64():
    g = torch.Generator().manual_seed(7)
    x = torch.randn(40, 24, generator=g, dtype=torch.float64)
    w = torch.randn(77, 24, generator=g, dtype=torch.float64) * 0.3
    b = torch.randn(77, generator=g, dtype=torch.float64)
    t = torch.randint(0, 77, (40,), generator=g)
    t[::5] = -100
    for red in ("mean", "sum"):
        for sc in (None, 3.0):
            kw = dict(bias=b, lse_square_scale=1e-2, label_smoothing=0.1, reduction=red, softcap=sc)
            res = flce_oracle(x, w, t, **kw)
            loss, z, gx, gw, gb = torch_linear_ce_reference(x, w, t, dtype=torch.float64, **kw)
            assert abs(float(res.loss) - float(loss)) < 1e-10 * max(1, abs(float(loss)))
            assert (res.grad_input - gx).abs().max() < 1e-11
            assert (res.grad_weight - gw).abs().max() < 1e-11
            assert (res.grad_bias - gb).abs().max() < 1e-11


# ---- stand-alone cross-entropy -----------------------------------------------------------------------------------
from golden_util import ce_golden_names  # noqa: E402
from oracle.flce_oracle import ce_oracle  # noqa: E402


@pytest.mark.parametrize("name", ce_golden_names())
def test_ce_oracle_matches_reference_golden(name):
    rec, meta = load_golden(name)
    bf16 = meta.get("dtype") == "bfloat16"
    logits, t = torch.from_numpy(rec["logits"]), torch.from_numpy(rec["target"])
    go = golden_grad_output(rec, meta)
    res = ce_oracle(logits, t, weight=None if "weight" not in rec else torch.from_numpy(rec["weight"]),
                    ignore_index=meta["ignore_index"], lse_square_scale=meta.get("lse_square_scale", 0.0),
                    label_smoothing=meta.get("label_smoothing", 0.0), reduction=meta.get("reduction", "mean"),
                    softcap=meta.get("softcap"), grad_output=go)
    # the reference keeps loss rows in the logits' dtype: bf16 rounding for the bf16 case
    atol, rtol = (0.0, 1e-2) if bf16 else (2e-5 * max(1.0, float(np.abs(rec["ref_loss"]).max())), 2e-4)
    _close(res.loss, rec["ref_loss"], atol, rtol, "loss")
    if "ref_z_loss" in rec:
        _close(res.z_loss, rec["ref_z_loss"], 2e-5, 2e-4, "z_loss")
    gmax = float(np.abs(rec["ref_grad_logits"]).max())
    _close(res.grad_input, rec["ref_grad_logits"], (8e-3 if bf16 else 2e-6) * gmax, 1e-2 if bf16 else 1e-3, "grad_logits")
    if "ref_token_accuracy" in rec:
        _close(res.token_accuracy, rec["ref_token_accuracy"], 1e-6, 0, "token_accuracy")
    if "ref_predicted_tokens" in rec:
        assert np.array_equal(res.predicted_tokens.numpy(), rec["ref_predicted_tokens"])


# ---------------------------------------------------------------- fused linear JSD / scaled cross-entropy oracles
def _jsd_inputs(rec, meta):
    t = {k: torch.from_numpy(rec[k]) for k in ("student_input", "student_weight", "teacher_input", "teacher_weight")}
    labels = torch.from_numpy(rec["labels"]) if "labels" in rec else None
    kw = dict(jsd_beta=meta.get("beta", 0.5), ignore_index=meta["ignore_index"], temperature=meta.get("temperature", 1.0))
    return t, labels, kw


@pytest.mark.parametrize("name", jsd_golden_names())
def test_jsd_oracle_matches_reference_golden(name):
    """fp64 closed form vs the reference's fused_linear_jsd_forward (/ _backward) run on CPU by Triton's interpreter."""
    rec, meta = load_golden(name)
    bf16 = meta.get("dtype") == "bfloat16"
    t, labels, kw = _jsd_inputs(rec, meta)
    low = torch.bfloat16 if bf16 else None
    res = fused_linear_jsd_oracle(t["student_input"], t["student_weight"], t["teacher_input"], t["teacher_weight"], labels,
                                  grad_output=meta.get("grad_output", 1.0), round_logits_to=low, round_dlogits_to=low, **kw)
    _close(res.loss, rec["ref_loss"], 1e-2 if bf16 else 1e-6, 1e-2 if bf16 else 2e-5, "loss")
    for key, got in (("ref_grad_input", res.grad_input), ("ref_grad_weight", res.grad_weight)):
        gmax = float(np.abs(rec[key]).max())
        _close(got, rec[key], (1e-2 if bf16 else 2e-6) * gmax, 2e-2 if bf16 else 2e-4, key)
    if "labels" in rec:
        ignored = rec["labels"] == meta["ignore_index"]
        assert float(np.abs(res.grad_input.numpy()[ignored]).max(initial=0.0)) == 0.0


@pytest.mark.parametrize("name", sce_golden_names())
def test_scaled_ce_oracle_matches_reference_golden(name):
    """fp64 closed form vs the reference's LigerFusedLinearScaledCrossEntropyFunction on CPU tensors."""
    rec, meta = load_golden(name)
    bf16 = meta.get("dtype") == "bfloat16"
    x, w, t = torch.from_numpy(rec["x"]), torch.from_numpy(rec["w"]), torch.from_numpy(rec["target"])
    g_nll = torch.from_numpy(rec["grad_nll"]) if meta["grads"] in ("both", "nll") else None
    g_ent = torch.from_numpy(rec["grad_entropy"]) if meta["grads"] in ("both", "entropy") else None
    low = torch.bfloat16 if bf16 else None
    res = fused_linear_scaled_ce_oracle(x, w, t, meta["temperature"], -100, g_nll, g_ent, round_logits_to=low, round_dlogits_to=low)
    _close(res.nll, rec["ref_nll"], 4e-2 if bf16 else 2e-5, 1e-2 if bf16 else 2e-5, "nll")
    _close(res.entropy, rec["ref_entropy"], 4e-2 if bf16 else 2e-5, 1e-2 if bf16 else 2e-5, "entropy")
    for key, got in (("ref_grad_input", res.grad_input), ("ref_grad_weight", res.grad_weight)):
        gmax = float(np.abs(rec[key]).max())
        _close(got, rec[key], (2e-2 if bf16 else 5e-6) * gmax, 2e-2 if bf16 else 5e-4, key)
    ignored = rec["target"] == -100
    assert float(np.abs(res.nll.numpy()[ignored]).max(initial=0.0)) == 0.0


def test_distill_oracles_equal_autograd_fp64():
    """Both closed forms against torch autograd in fp64 (independent of the reference's hand-written gradients)."""
    g = torch.Generator().manual_seed(11)
    N, H, V = 13, 9, 29
    xs = torch.randn(N, H, generator=g, dtype=torch.float64).requires_grad_(True)
    ws = torch.randn(V, H, generator=g, dtype=torch.float64).requires_grad_(True)
    xt, wt = torch.randn(N, 2 * H, generator=g, dtype=torch.float64), torch.randn(V, 2 * H, generator=g, dtype=torch.float64)
    labels = torch.randint(0, V, (N,), generator=g)
    labels[::4] = -100
    for beta in (0.0, 0.3, 1.0):
        X = torch.log_softmax(xs @ ws.T / 1.7, -1)
        Y = torch.log_softmax(xt @ wt.T / 1.7, -1)
        P, Q = Y.exp(), X.exp()
        if beta == 0.0:
            rows = (P * (Y - X)).sum(-1)
        elif beta == 1.0:
            rows = (Q * (X - Y)).sum(-1)
        else:
            M = beta * P + (1 - beta) * Q
            rows = beta * (P * (Y - M.log())).sum(-1) + (1 - beta) * (Q * (X - M.log())).sum(-1)
        live = labels != -100
        loss = (rows * live).sum() / live.sum()
        gx, gw = torch.autograd.grad(loss, (xs, ws))
        res = fused_linear_jsd_oracle(xs.detach(), ws.detach(), xt, wt, labels, jsd_beta=beta, temperature=1.7)
        _close(res.loss, loss.detach(), 1e-12, 1e-10, "jsd loss")
        _close(res.grad_input, gx, 1e-12, 1e-9, "jsd grad_input")
        _close(res.grad_weight, gw, 1e-12, 1e-9, "jsd grad_weight")
    s = xs @ ws.T / 0.8
    logp = torch.log_softmax(s, -1)
    nll = -logp.gather(-1, labels.clamp_min(0)[:, None])[:, 0]
    ent = -(logp.exp() * logp).sum(-1)
    g_nll, g_ent = torch.randn(N, generator=g, dtype=torch.float64), torch.randn(N, generator=g, dtype=torch.float64)
    live = (labels != -100).double()
    gx, gw = torch.autograd.grad(((nll * g_nll + ent * g_ent) * live).sum(), (xs, ws))
    res = fused_linear_scaled_ce_oracle(xs.detach(), ws.detach(), labels, 0.8, -100, g_nll, g_ent)
    _close(res.nll, (nll * live).detach(), 1e-12, 1e-10, "nll")
    _close(res.entropy, (ent * live).detach(), 1e-12, 1e-10, "entropy")
    _close(res.grad_input, gx, 1e-12, 1e-9, "sce grad_input")
    _close(res.grad_weight, gw, 1e-12, 1e-9, "sce grad_weight")
