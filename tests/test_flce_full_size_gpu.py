"""Behaviour around the core operator, kept in a file of its own that is collected after the core parity files:
automatic mixed precision (fp32 parameters and inputs under torch.autocast) and the out-of-range-target report."""

import pytest
import torch

import flce_cases
from flce_cases import make_inputs, oracle_for
from test_flce_gpu import _check

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("amp_dtype", [torch.bfloat16, torch.float16])
def test_amp_autocast_with_fp32_parameters(amp_dtype):
    """fp32 master weights and inputs under torch.autocast: operands are cast to the autocast dtype, gradients come back
    in fp32 (reference: test/transformers/test_fused_linear_cross_entropy.py:558-604)."""
    from liger_kernel_b200 import LigerFusedLinearCrossEntropyLoss

    dev = flce_cases.DEVICE
    x, w, t, b, _ = make_inputs(256, 128, 1000, torch.float32, seed=31, bias=True)
    xd = x.to(dev).clone().requires_grad_(True)
    wd = w.to(dev).clone().requires_grad_(True)
    bd = b.to(dev).clone().requires_grad_(True)
    with torch.autocast(device_type="cuda", dtype=amp_dtype):
        loss = LigerFusedLinearCrossEntropyLoss()(wd, xd, t.to(dev), bd)
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

    dev = flce_cases.DEVICE
    x, w, t, _, _ = make_inputs(200, 64, 300, torch.bfloat16, seed=41)
    t[5], t[9] = 303, -7
    prep = mod._Prepared(x.to(dev), w.to(dev), t.to(dev), None, None, -100, 0.0, 0.0, "mean", None, False)
    out, norm, _ = mod.flce_forward_device(prep)
    assert int(norm[3].item()) == 2 and bool(torch.isfinite(out["scalars"][0]))
    monkeypatch.setattr(mod, "CHECK_TARGETS", True)
    with pytest.raises(AssertionError, match="out of bounds"):
        mod.LigerFusedLinearCrossEntropyFunction.apply(x.to(dev), w.to(dev), t.to(dev))
    t[5], t[9] = 1, 2
    mod.LigerFusedLinearCrossEntropyFunction.apply(x.to(dev), w.to(dev), t.to(dev))


FULL_SIZE = {
    # the benchmark configurations 3-5 at their full sizes (configuration 2 is covered by test_flce_gpu.py::test_full_size_properties)
    "c3_qwen_style": (32768, 3584, 152064, 0.20, dict(label_smoothing=0.1, lse_square_scale=1e-4)),
    "c4_gemma_style": (16384, 3584, 256000, 0.05, dict(softcap=30.0, reduction="sum")),
    "c5_llama70b_head": (65536, 8192, 128256, 0.05, dict()),
}


@pytest.mark.parametrize("name", sorted(FULL_SIZE))
def test_full_size_configs_sampled_against_fp64(name):
    """Full-size heads: loss consistency, exact zeros on ignored rows, and sampled rows of lse / grad_input / grad_weight
    against fp64 math streamed over the whole vocabulary and all tokens."""
    import liger_kernel_b200.ops.fused_linear_cross_entropy as mod
    from flce_cases import sampled_fp64_check

    N, H, V, ign, kw = FULL_SIZE[name]
    dev = flce_cases.DEVICE
    if dev == "cuda" and torch.cuda.get_device_properties(0).total_memory < 60e9:
        pytest.skip("needs ~25 GB of device memory")
    g = torch.Generator(device=dev).manual_seed(77)
    x = torch.randn(N, H, generator=g, device=dev).bfloat16()
    w = (torch.randn(V, H, generator=g, device=dev) * 0.02).bfloat16()
    t = torch.randint(0, V, (N,), generator=g, device=dev)
    t[torch.rand(N, generator=g, device=dev) < ign] = -100
    red = kw.get("reduction", "mean")
    xd, wd = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    loss = mod.LigerFusedLinearCrossEntropyFunction.apply(
        xd, wd, t, None, None, -100, kw.get("lse_square_scale", 0.0), kw.get("label_smoothing", 0.0), red, kw.get("softcap"))[0]
    loss.backward()
    prep = mod._Prepared(x, w, t, None, None, -100, kw.get("lse_square_scale", 0.0), kw.get("label_smoothing", 0.0), red,
                         kw.get("softcap"), False, want_argmax=False)
    out, norm, _ = mod.flce_forward_device(prep)
    n_valid = int((t != -100).sum())
    assert int(norm[0].item()) == n_valid
    # the scalar loss is the ordered sum of the per-row losses; ignored rows contribute exact zeros everywhere
    assert abs(float(out["loss_rows"].double().sum()) - float(loss.detach())) <= 1e-5 * abs(float(loss.detach()))
    assert float(out["loss_rows"][t == -100].abs().max()) == 0.0 and float(xd.grad[t == -100].abs().max()) == 0.0
    sampled_fp64_check(x, w, t, out["lse"], xd.grad, wd.grad, vocab_samples=(0, 1, 4097, V // 2), **kw)
