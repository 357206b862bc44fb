"""Behaviour around the core operator, kept in a file of its own that is collected after the core parity files:
automatic mixed precision (fp32 parameters and inputs under torch.autocast) and the out-of-range-target report."""

import pytest
import torch

from flce_cases import make_inputs, oracle_for
from test_flce_gpu import _check

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("amp_dtype", [torch.bfloat16, torch.float16])
def test_amp_autocast_with_fp32_parameters(amp_dtype):
    """fp32 master weights and inputs under torch.autocast: operands are cast to the autocast dtype, gradients come back
    in fp32 (reference: test/transformers/test_fused_linear_cross_entropy.py:558-604)."""
    from liger_kernel_b200 import LigerFusedLinearCrossEntropyLoss

    x, w, t, b, _ = make_inputs(256, 128, 1000, torch.float32, seed=31, bias=True)
    xd = x.cuda().requires_grad_(True)
    wd = w.cuda().requires_grad_(True)
    bd = b.cuda().requires_grad_(True)
    with torch.autocast(device_type="cuda", dtype=amp_dtype):
        loss = LigerFusedLinearCrossEntropyLoss()(wd, xd, t.cuda(), bd)
    loss.backward()
    assert loss.dtype == torch.float32 and xd.grad.dtype == torch.float32 and wd.grad.dtype == torch.float32
    assert bd.grad.dtype == torch.float32
    ora = oracle_for(x.to(amp_dtype), w.to(amp_dtype), t, bias=b.to(amp_dtype))
    res = dict(loss=loss.detach().cpu(), z_loss=torch.zeros(()), predicted_tokens=ora.predicted_tokens,
               grad_input=xd.grad.cpu(), grad_weight=wd.grad.cpu(), grad_bias=bd.grad.cpu())
    _check(res, ora, amp_dtype, "mean", 256)


def test_out_of_range_targets_are_counted_and_optionally_raised(monkeypatch):
    """Targets that are neither ignore_index nor a class id never touch memory; they are counted on the device and a caller
    can ask for the reference's assertion (ops/cross_entropy.py:389-392) at the price of a host synchronisation."""
    import liger_kernel_b200.ops.fused_linear_cross_entropy as mod

    x, w, t, _, _ = make_inputs(200, 64, 300, torch.bfloat16, seed=41)
    t[5], t[9] = 303, -7
    prep = mod._Prepared(x.cuda(), w.cuda(), t.cuda(), None, None, -100, 0.0, 0.0, "mean", None, False)
    out, norm, _ = mod.flce_forward_device(prep)
    assert int(norm[3].item()) == 2 and bool(torch.isfinite(out["scalars"][0]))
    monkeypatch.setattr(mod, "CHECK_TARGETS", True)
    with pytest.raises(AssertionError, match="out of bounds"):
        mod.LigerFusedLinearCrossEntropyFunction.apply(x.cuda(), w.cuda(), t.cuda())
    t[5], t[9] = 1, 2
    mod.LigerFusedLinearCrossEntropyFunction.apply(x.cuda(), w.cuda(), t.cuda())
