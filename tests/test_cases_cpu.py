"""The sampled fp64 checker used by the full-size GPU tests, exercised on the CPU against the oracle: fed with the
oracle's own lse and gradients it must accept them for every feature combination, and it must reject a perturbed result."""

import pytest
import torch

from flce_cases import make_inputs, oracle_for, sampled_fp64_check


@pytest.mark.parametrize("kw", [dict(), dict(label_smoothing=0.1, lse_square_scale=1e-2), dict(softcap=3.0, reduction="sum"),
                                dict(label_smoothing=0.2, softcap=5.0, lse_square_scale=1e-3)])
def test_sampled_checker_accepts_oracle_and_rejects_errors(kw):
    x, w, t, _, _ = make_inputs(300, 40, 517, torch.float32, seed=5, ignore_frac=0.2, wscale=0.4)
    ora = oracle_for(x, w, t, **kw)
    lse = torch.where(t != -100, ora.lse, torch.logsumexp((x.double() @ w.double().t()) if kw.get("softcap") is None else
                                                         kw["softcap"] * torch.tanh(x.double() @ w.double().t() / kw["softcap"]), 1))
    args = dict(n_row_samples=50, vocab_samples=(0, 3, 200), row_chunk=64, vocab_chunk=100, **kw)
    err = sampled_fp64_check(x, w, t, lse.float(), ora.grad_input.float(), ora.grad_weight.float(), **args)
    assert err <= 1e-6
    bad = ora.grad_weight.float().clone()
    bad[200] *= 1.5
    with pytest.raises(AssertionError, match="grad_weight rows"):
        sampled_fp64_check(x, w, t, lse.float(), ora.grad_input.float(), bad, **args)
    with pytest.raises(AssertionError, match="lse error"):
        sampled_fp64_check(x, w, t, lse.float() + 1e-3, ora.grad_input.float(), ora.grad_weight.float(), **args)
