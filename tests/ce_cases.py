"""Shared bodies of the stand-alone cross-entropy tests: the same cases run on a B200 (tests/test_y_cross_entropy_gpu.py)
and, with the library's SIMT kernels emulated on the host, on CPU tensors (tests/test_simt_emulation_cpu.py)."""

import numpy as np
import pytest
import torch

from flce_cases import assert_close
from golden_util import golden_grad_output, load_golden
from oracle.flce_oracle import ce_oracle

FEATURES = [dict(), dict(label_smoothing=0.1), dict(lse_square_scale=1e-3), dict(softcap=30.0),
            dict(label_smoothing=0.1, ignore_index=42, lse_square_scale=1e-4, softcap=30.0)]


def run_ce(logits, t, device, weight=None, grad_output=None, inplace=False, **kw):
    import liger_kernel_b200.ops.cross_entropy as mod
    from liger_kernel_b200.ops.cross_entropy import LigerCrossEntropyFunction as Fn

    before = mod.INPLACE_GRADIENT
    mod.INPLACE_GRADIENT = inplace
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
        mod.INPLACE_GRADIENT = before
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


def case_correctness(device, N, V, dtype, reduction, feat):
    logits, t = random_case(N, V, dtype, feat)
    kw = dict(reduction=reduction, **feat)
    check_ce(run_ce(logits, t, device, **kw), ce_oracle(logits, t, **kw), dtype)


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
