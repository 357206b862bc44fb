"""Shared helpers for the FLCE parity tests: seeded inputs and comparison against the CPU oracle."""

import numpy as np
import torch

from oracle.flce_oracle import flce_oracle


def make_inputs(N, H, V, dtype, seed=0, ignore_frac=0.1, ignore_index=-100, wscale=None, bias=False, ce_weight=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, H, generator=g).to(dtype)
    w = (torch.randn(V, H, generator=g) * (wscale if wscale is not None else H ** -0.5)).to(dtype)
    t = torch.randint(0, V, (N,), generator=g)
    if ignore_index >= 0:
        t[t == ignore_index] = (ignore_index + 1) % V
    t[torch.rand(N, generator=g) < ignore_frac] = ignore_index
    b = (torch.randn(V, generator=g) * 0.5).to(dtype) if bias else None
    cw = (torch.rand(V, generator=g) + 0.5) if ce_weight else None
    return x, w, t, b, cw


def run_cuda(x, w, t, bias=None, ce_weight=None, grad_output=None, want_grads=True, **kw):
    """Public-API call on the GPU; returns a dict of CPU tensors."""
    from liger_kernel_b200.ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction as Fn

    xd = x.cuda().requires_grad_(want_grads)
    wd = w.cuda().requires_grad_(want_grads)
    bd = None if bias is None else bias.cuda().requires_grad_(want_grads)
    cwd = None if ce_weight is None else ce_weight.cuda()
    loss, z, acc, pred = Fn.apply(
        xd, wd, t.cuda(), bd, cwd, kw.get("ignore_index", -100), kw.get("lse_square_scale", 0.0),
        kw.get("label_smoothing", 0.0), kw.get("reduction", "mean"), kw.get("softcap"), True, None,
        kw.get("use_token_scaling", False), True, True,
    )
    out = dict(loss=loss.detach().cpu(), z_loss=z.detach().cpu(), token_accuracy=acc.detach().cpu(),
               predicted_tokens=pred.cpu())
    if want_grads:
        if grad_output is None:
            go = torch.ones_like(loss)
        else:
            go = torch.as_tensor(grad_output, dtype=loss.dtype).cuda().expand_as(loss).contiguous()
        loss.backward(go)
        out["grad_input"] = xd.grad.cpu()
        out["grad_weight"] = wd.grad.cpu()
        out["grad_bias"] = None if bd is None else bd.grad.cpu()
    return out


def oracle_for(x, w, t, bias=None, ce_weight=None, grad_output=None, **kw):
    return flce_oracle(
        x, w, t, bias=bias, ce_weight=ce_weight, ignore_index=kw.get("ignore_index", -100),
        lse_square_scale=kw.get("lse_square_scale", 0.0), label_smoothing=kw.get("label_smoothing", 0.0),
        reduction=kw.get("reduction", "mean"), softcap=kw.get("softcap"),
        use_token_scaling=kw.get("use_token_scaling", False), grad_output=grad_output,
    )


def assert_close(got, want, atol, rtol, what):
    got = np.asarray(got.detach().double().cpu() if torch.is_tensor(got) else got, dtype=np.float64)
    want = np.asarray(want.detach().double().cpu() if torch.is_tensor(want) else want, dtype=np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    excess = np.abs(got - want) - (atol + rtol * np.abs(want))
    assert np.all(excess <= 0), (
        f"{what}: {int((excess > 0).sum())}/{excess.size} out of tolerance, max |diff| {np.abs(got - want).max():.3e}, "
        f"max |want| {np.abs(want).max():.3e}"
    )
