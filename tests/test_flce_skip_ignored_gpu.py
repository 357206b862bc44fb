"""LIGER_B200_FLCE_SKIP_IGNORED: rows whose target is ignore_index are moved to the end on the device and the sweeps
skip the token tiles that hold only such rows.  Results must equal the plain path (loss to rounding of the summation
order, gradients to a 16-bit ulp) and the oracle, for any ignored fraction including none and all."""

import pytest
import torch

from flce_cases import assert_close, make_inputs, oracle_for, run_cuda
from test_flce_gpu import _check

pytestmark = pytest.mark.gpu


@pytest.fixture
def skipping(monkeypatch):
    import liger_kernel_b200.ops.fused_linear_cross_entropy as mod

    monkeypatch.setattr(mod, "SKIP_IGNORED", True)
    return mod


@pytest.mark.parametrize("ignore_frac", [0.0, 0.05, 0.5, 0.97])
@pytest.mark.parametrize("N,H,V", [(1000, 256, 3000), (4096, 512, 8192), (300, 31, 123)])
def test_skip_ignored_matches_oracle_and_plain_path(skipping, monkeypatch, N, H, V, ignore_frac):
    x, w, t, b, _ = make_inputs(N, H, V, torch.bfloat16, seed=N + V, ignore_frac=ignore_frac, bias=True)
    kw = dict(label_smoothing=0.1, lse_square_scale=1e-4)
    fast = run_cuda(x, w, t, bias=b, **kw)
    _check(fast, oracle_for(x, w, t, bias=b, **kw), torch.bfloat16, "mean", N)
    monkeypatch.setattr(skipping, "SKIP_IGNORED", False)
    plain = run_cuda(x, w, t, bias=b, **kw)
    assert_close(fast["loss"], plain["loss"], 0, 1e-6, "loss")
    assert torch.equal(fast["predicted_tokens"], plain["predicted_tokens"])
    assert_close(fast["grad_input"].float(), plain["grad_input"].float(), 1e-9, 1e-2, "grad_input")
    assert_close(fast["grad_weight"].float(), plain["grad_weight"].float(), 8e-3 * float(plain["grad_weight"].abs().max()), 2e-2, "grad_weight")
    assert float(fast["grad_input"][t == -100].abs().max() if (t == -100).any() else 0.0) == 0.0


def test_skip_ignored_all_rows_ignored_and_per_token_gradient(skipping):
    x, w, t, _, _ = make_inputs(512, 128, 1000, torch.bfloat16, seed=3, ignore_frac=1.1)
    res = run_cuda(x, w, t)
    assert float(res["loss"]) == 0.0
    assert float(res["grad_input"].abs().max()) == 0.0 and float(res["grad_weight"].abs().max()) == 0.0
    x, w, t, _, _ = make_inputs(700, 96, 500, torch.bfloat16, seed=7, ignore_frac=0.3)
    go = torch.rand(700) + 0.5
    res = run_cuda(x, w, t, reduction="none", grad_output=go)
    ora = oracle_for(x, w, t, reduction="none", grad_output=go)
    assert_close(res["loss"], ora.loss.float(), 1e-4, 1e-4, "loss rows")
    for key, want in (("grad_input", ora.grad_input), ("grad_weight", ora.grad_weight)):      # un-normalised rows: scale-aware bound
        assert_close(res[key].float(), want.float(), 8e-3 * float(want.abs().max()), 5e-2, key)
