"""Shared bodies of the stand-alone cross-entropy tests: the same cases run on a B200 (tests/test_cross_entropy_gpu.py)
and, with the library's SIMT kernels emulated on the host, on CPU tensors (tests/test_simt_emulation_cpu.py)."""

import numpy as np
import pytest
import torch

from flce_cases import assert_close
from golden_util import golden_grad_output, load_golden
from oracle.flce_oracle import ce_oracle

FEATURES = [dict(), dict(label_smoothing=0.1), dict(lse_square_scale=1e-3), dict(softcap=30.0),
            dict(label_smoothing=0.1, ignore_index=42, lse_square_scale=1e-4, softcap=30.0)]


def run_ce(logits, t, device, weight=None, grad_output=None, inplace=False, mode=None, **kw):
    import liger_kernel_b200.ops.cross_entropy as mod
    from liger_kernel_b200.ops.cross_entropy import LigerCrossEntropyFunction as Fn

    before, mode_before = mod.INPLACE_GRADIENT, mod.MODE
    mod.INPLACE_GRADIENT = inplace
    if mode is not None:
        mod.MODE = mode
    try:
        x = logits.to(device).clone().requires_grad_(True)
        loss, z, acc, pred = Fn.apply(x, t.to(device), None if weight is None else weight.to(device), kw.get("ignore_index", -100),
                                      kw.get("lse_square_scale", 0.0), kw.get("label_smoothing", 0.0),
                                      kw.get("reduction", "mean"), kw.get("softcap"), True, True, True)
        if grad_output is None:
            go = torch.ones_like(loss)
        else:
            go = torch.as_tensor(grad_output, dtype=loss.dtype).to(device).expand_as(loss).contiguous()
        loss.backward(go)
    finally:
        mod.INPLACE_GRADIENT, mod.MODE = before, mode_before
    return dict(loss=loss.detach().float().cpu(), z_loss=z.float().cpu(), token_accuracy=acc.cpu(), predicted=pred.cpu(),
                grad=x.grad.float().cpu())


def check_ce(res, ora, dtype):
    low = dtype != torch.float32
    scale = max(1.0, float(ora.loss.abs().max()))
    assert_close(res["loss"], ora.loss.float(), (1e-2 if low else 1e-5) * scale, 1e-2 if low else 2e-5, "loss")
    assert torch.equal(res["predicted"], ora.predicted_tokens)
    gmax = float(ora.grad_input.abs().max())
    assert_close(res["grad"], ora.grad_input.float(), (8e-3 if low else 2e-6) * max(gmax, 1e-30), 2e-2 if low else 2e-4, "grad")


def random_case(N, V, dtype, feat):
    g = torch.Generator().manual_seed(N + V)
    logits = (torch.randn(N, V, generator=g) * 2).to(dtype)
    t = torch.randint(0, V, (N,), generator=g)
    ii = feat.get("ignore_index", -100)
    if ii >= 0:
        t[t == ii] = ii + 1
    t[torch.rand(N, generator=g) < 0.1] = ii
    return logits, t


def case_correctness(device, N, V, dtype, reduction, feat, mode=None):
    logits, t = random_case(N, V, dtype, feat)
    kw = dict(reduction=reduction, **feat)
    check_ce(run_ce(logits, t, device, mode=mode, **kw), ce_oracle(logits, t, **kw), dtype)


def case_weights_none_reduction_upstream_gradient_and_inplace(device, N=300, V=1000):
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(N, V, generator=g) * 3
    t = torch.randint(0, V, (N,), generator=g)
    t[::7] = -100
    w = torch.rand(V, generator=g) + 0.5
    for kw, go in ((dict(label_smoothing=0.1), 2.0), (dict(reduction="none"), torch.rand(N) + 0.5), (dict(reduction="sum"), None)):
        res = run_ce(logits, t, device, weight=w, grad_output=go, **kw)
        check_ce(res, ce_oracle(logits, t, weight=w, grad_output=go, **kw), torch.float32)
    # in-place mode: the gradient lands in the logits' own storage, and a second backward is refused
    import liger_kernel_b200.ops.cross_entropy as mod
    from liger_kernel_b200.ops.cross_entropy import LigerCrossEntropyFunction as Fn

    base = logits.to(device)
    x = base.clone().requires_grad_(True)
    holder = x * 1.0                       # a non-leaf, as the output of an lm_head would be
    loss = Fn.apply(holder, t.to(device), None)[0]
    loss.backward(retain_graph=True)
    assert_close(x.grad.float().cpu(), ce_oracle(logits, t).grad_input.float(), 1e-7, 2e-4, "in-place grad")
    assert holder.data_ptr() != base.data_ptr() and not torch.equal(holder.detach(), base)   # overwritten by the gradient
    with pytest.raises(RuntimeError, match="overwritten"):
        loss.backward()
    assert mod.INPLACE_GRADIENT is True


def case_all_ignored_is_exact_zero(device, N=64, V=500):
    logits = torch.randn(N, V).bfloat16()
    t = torch.full((N,), -100)
    res = run_ce(logits, t, device)
    assert float(res["loss"]) == 0.0 and float(res["grad"].abs().max()) == 0.0 and torch.all(res["predicted"] == -1)


def case_reference_golden(device, name):
    rec, meta = load_golden(name)
    dtype = getattr(torch, meta.get("dtype", "float32"))
    logits, t = torch.from_numpy(rec["logits"]).to(dtype), torch.from_numpy(rec["target"])
    w = None if "weight" not in rec else torch.from_numpy(rec["weight"])
    kw = dict(ignore_index=meta["ignore_index"], lse_square_scale=meta.get("lse_square_scale", 0.0),
              label_smoothing=meta.get("label_smoothing", 0.0), reduction=meta.get("reduction", "mean"), softcap=meta.get("softcap"))
    res = run_ce(logits, t, device, weight=w, grad_output=golden_grad_output(rec, meta), **kw)
    low = dtype != torch.float32
    want = torch.from_numpy(rec["ref_grad_logits"])
    assert_close(res["grad"], want, (8e-3 if low else 5e-6) * float(want.abs().max()), 2e-2 if low else 1e-3, "grad vs reference")
    assert_close(res["loss"], torch.from_numpy(rec["ref_loss"]), 0.0 if low else 2e-5 * max(1.0, float(np.abs(rec["ref_loss"]).max())),
                 1e-2 if low else 2e-4, "loss vs reference")


def case_true_class_gradient_confident_predictions(device, dtype, label_smoothing, reduction):
    """The reference's test of the same name (test/transformers/test_cross_entropy.py:1282-1324): once the model is confident,
    dx_y = (softmax(x_y) - (1 - label_smoothing)) / N is a small difference of large terms and must be formed before rounding to
    the logits' dtype.  Required: no less accurate than torch's own low-precision backward (within a factor of 4)."""
    import liger_kernel_b200 as lk

    torch.manual_seed(0)
    n, v = 96, 4096
    logits = torch.randn(n, v)
    target = torch.randint(0, v, (n,))
    logits[torch.arange(n), target] = logits.max(dim=-1).values + 10.0
    low = logits.to(dtype)
    ours = low.to(device).clone().requires_grad_(True)
    theirs = low.clone().requires_grad_(True)
    exact = low.clone().float().requires_grad_(True)
    torch_ce = torch.nn.CrossEntropyLoss(reduction=reduction, label_smoothing=label_smoothing)
    torch_ce(theirs, target).backward()
    torch_ce(exact, target).backward()
    lk.LigerCrossEntropyLoss(reduction=reduction, label_smoothing=label_smoothing)(ours, target.to(device)).backward()
    rows = torch.arange(n)
    ref = exact.grad[rows, target].double()
    torch_err = float((theirs.grad[rows, target].double() - ref).abs().max())
    our_err = float((ours.grad.cpu()[rows, target].double() - ref).abs().max())
    assert our_err <= max(4 * torch_err, torch.finfo(dtype).tiny), (our_err, torch_err)


def case_forward_only_structured_output_and_target_check(device):
    """No-grad forward (test_correctness_with_forward_only), the CrossEntropyOutput convention of the module
    (test_liger_cross_entropy_structured_output) and the optional out-of-range-target assertion
    (test_correctness_with_out_of_bounds_target_once)."""
    import liger_kernel_b200 as lk
    import liger_kernel_b200.ops.fused_linear_cross_entropy as fl

    logits, t = random_case(50, 300, torch.bfloat16, dict())
    with torch.no_grad():
        loss = lk.LigerCrossEntropyLoss()(logits.to(device), t.to(device))
    assert torch.is_tensor(loss) and loss.shape == () and not loss.requires_grad
    assert_close(loss.float().cpu(), ce_oracle(logits, t).loss.float(), 1e-2, 1e-2, "loss")
    out = lk.LigerCrossEntropyLoss(lse_square_scale=1e-3, return_z_loss=True, return_token_accuracy=True,
                                   return_predicted_tokens=True)(logits.to(device), t.to(device))
    assert isinstance(out, lk.CrossEntropyOutput)
    assert out.z_loss is not None and out.token_accuracy is not None and out.predicted_tokens.shape == (50,)
    bad = t.clone()
    bad[3] = 300
    before = fl.CHECK_TARGETS
    fl.CHECK_TARGETS = True
    try:
        with pytest.raises(AssertionError, match="out of bounds"):
            lk.LigerCrossEntropyLoss()(logits.to(device), bad.to(device))
        lk.LigerCrossEntropyLoss()(logits.to(device), t.to(device))
    finally:
        fl.CHECK_TARGETS = before
