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


# Where run_cuda puts its tensors.  The CPU suite switches this to "cpu" while the library handle is replaced by the
# kernel emulation (tests/emu_lib.py), so that the same test bodies run without a GPU.
DEVICE = "cuda"


def run_cuda(x, w, t, bias=None, ce_weight=None, grad_output=None, want_grads=True, **kw):
    """Public-API call on the GPU; returns a dict of CPU tensors."""
    from liger_kernel_b200.ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction as Fn

    dev = DEVICE
    xd = x.to(dev).clone().requires_grad_(want_grads)
    wd = w.to(dev).clone().requires_grad_(want_grads)
    bd = None if bias is None else bias.to(dev).clone().requires_grad_(want_grads)
    cwd = None if ce_weight is None else ce_weight.to(dev)
    loss, z, acc, pred = Fn.apply(
        xd, wd, t.to(dev), bd, cwd, kw.get("ignore_index", -100), kw.get("lse_square_scale", 0.0),
        kw.get("label_smoothing", 0.0), kw.get("reduction", "mean"), kw.get("softcap"), True, None,
        kw.get("use_token_scaling", False), True, True,
    )
    out = dict(loss=loss.detach().cpu(), z_loss=z.detach().cpu(), token_accuracy=acc.detach().cpu(),
               predicted_tokens=pred.cpu())
    if want_grads:
        if grad_output is None:
            go = torch.ones_like(loss)
        else:
            go = torch.as_tensor(grad_output, dtype=loss.dtype).to(dev).expand_as(loss).contiguous()
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


def sampled_fp64_check(x, w, t, lse, grad_input, grad_weight, *, reduction="mean", label_smoothing=0.0, lse_square_scale=0.0,
                       softcap=None, ignore_index=-100, n_row_samples=64, vocab_samples=(0, 1, 4097), row_chunk=8192,
                       vocab_chunk=16384):
    """Size-independent check of a full-size result against fp64 math on a sample, on whatever device the tensors live:
    * for sampled token rows: lse and the row of grad_input, from the whole vocabulary (streamed in chunks);
    * for sampled vocabulary rows: the row of grad_weight, from all tokens (streamed in chunks), using the per-row lse
      under test (which the first part validates on its sample).
    Returns the largest relative lse error seen; raises AssertionError on a mismatch."""
    N, H = x.shape
    V = w.shape[0]
    dev = x.device
    alpha, lam = float(label_smoothing), float(lse_square_scale)
    eps = alpha / V
    valid = t != ignore_index
    n_valid = int(valid.sum())
    inv_n = 1.0 / n_valid if reduction == "mean" else 1.0

    def capped(z):
        if softcap is None:
            return z, torch.ones_like(z)
        th = torch.tanh(z / softcap)
        return softcap * th, 1 - th * th

    # ---- sampled token rows
    rows = torch.arange(0, N, max(1, N // n_row_samples), device=dev)[:n_row_samples]
    xr = x[rows].double()
    s_parts, chain_parts = [], []
    for v0 in range(0, V, vocab_chunk):
        s, ch = capped(xr @ w[v0:v0 + vocab_chunk].double().t())
        s_parts.append(s)
        chain_parts.append(ch)
    s = torch.cat(s_parts, dim=1)
    chain = torch.cat(chain_parts, dim=1)
    lse_ref = torch.logsumexp(s, dim=1)
    lse_err = float(((lse[rows].double() - lse_ref).abs() / lse_ref.abs().clamp(min=1.0)).max())
    assert lse_err <= 1e-5, f"lse error {lse_err:.3e}"
    tr = t[rows]
    vr = valid[rows]
    g = torch.exp(s - lse_ref[:, None]) * (1 + 2 * lam * lse_ref)[:, None] - eps
    hit_rows = torch.arange(len(rows), device=dev)[vr]
    g[hit_rows, tr[vr]] -= (1 - alpha)
    g = g * chain * (vr.double() * inv_n)[:, None]
    dx_ref = torch.zeros(len(rows), H, dtype=torch.float64, device=dev)
    for v0 in range(0, V, vocab_chunk):
        dx_ref += g[:, v0:v0 + vocab_chunk] @ w[v0:v0 + vocab_chunk].double()
    assert_close(grad_input[rows].float().cpu(), dx_ref.float().cpu(), 8e-3 * float(dx_ref.abs().max()), 5e-2, "grad_input rows")

    # ---- sampled vocabulary rows
    vs = torch.tensor([v for v in vocab_samples if v < V] + [V - 1], device=dev)
    wv = w[vs].double()
    dw_ref = torch.zeros(len(vs), H, dtype=torch.float64, device=dev)
    for r0 in range(0, N, row_chunk):
        xc = x[r0:r0 + row_chunk].double()
        lc = lse[r0:r0 + row_chunk].double()
        sc, chc = capped(xc @ wv.t())
        gc = torch.exp(sc - lc[:, None]) * (1 + 2 * lam * lc)[:, None] - eps
        gc = gc - (1 - alpha) * (t[r0:r0 + row_chunk, None] == vs[None, :]).double()
        gc = gc * chc * (valid[r0:r0 + row_chunk].double() * inv_n)[:, None]
        dw_ref += gc.t() @ xc
    assert_close(grad_weight[vs].float().cpu(), dw_ref.float().cpu(), 8e-3 * float(dw_ref.abs().max()), 5e-2, "grad_weight rows")
    return lse_err
