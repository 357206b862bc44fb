"""The CPU oracle against the golden vectors produced by the reference itself.

Mirrors the comparisons of test/transformers/test_fused_linear_cross_entropy.py
(reference) with stored outputs instead of a live GPU run.
"""

import numpy as np
import pytest
import torch

from golden_util import golden_grad_output, golden_kwargs, golden_names, load_golden
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
