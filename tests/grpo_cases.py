"""Shared body of the GRPO tests: the library's operator on the GPU (tests/test_grpo_gpu.py) or on the host emulation
(tests/test_grpo_emulation_cpu.py) against torch in float64 with materialised logits, written the way GRPOTrainer and the
reference's test (test/chunked_loss/test_grpo_loss.py: TorchLMHeadGRPO) write it."""

import math

import torch
import torch.nn.functional as F

from flce_cases import assert_close


def torch_grpo(x, w, ids, mask, adv, ref=None, old=None, beta=0.04, eps_lo=0.2, eps_hi=0.2, loss_type="dapo",
               max_len=None, level="token", temperature=1.0, delta=None, bias_corr=False):
    x = x.double().requires_grad_(True)
    w = w.double().requires_grad_(True)
    maskf = mask.double()

    def logps(xx, ww):
        lp = F.log_softmax((xx @ ww.t()) / temperature, dim=-1)
        return torch.gather(lp, 2, ids.unsqueeze(2)).squeeze(2)

    lp = logps(x, w)
    ref_lp = logps(ref[0].double(), ref[1].double()).detach() if ref is not None else lp.detach()
    old_lp = old.double() if old is not None else lp.detach()
    log_ratio = lp - old_lp
    if level == "sequence":
        log_ratio = ((log_ratio * maskf).sum(-1) / maskf.sum(-1).clamp(min=1)).unsqueeze(-1)
    c1 = torch.exp(log_ratio)
    a = adv.double().unsqueeze(1)
    if loss_type == "vespo":
        with torch.no_grad():
            seq = (torch.clamp(lp - old_lp, -20, 20) * maskf).sum(-1, keepdim=True).clamp(math.log(1e-8), 20.0)
            pos = a >= 0
            k, lam = torch.where(pos, 2.0, 3.0), torch.where(pos, 3.0, 2.0)
            phi = torch.exp(lam + k * seq - lam * torch.exp(seq))
        per_token = -phi * a * lp
    elif loss_type == "cispo":
        per_token = -torch.clamp(c1, max=eps_hi).detach() * a * lp
    else:
        c2 = torch.clamp(c1, 1 - eps_lo, 1 + eps_hi)
        c1d = c1 if delta is None else torch.clamp(c1, max=delta)
        per_token = -torch.min(c1d * a, c2 * a)
    if beta != 0:
        kl = torch.exp(ref_lp - lp) - (ref_lp - lp) - 1
        if bias_corr:
            kl = kl * torch.exp(log_ratio)
        per_token = per_token + beta * kl
    if loss_type == "grpo":
        loss = ((per_token * maskf).sum(-1) / maskf.sum(-1).clamp(min=1)).mean()
    elif loss_type == "bnpo":
        loss = (per_token * maskf).sum() / maskf.sum().clamp(min=1)
    elif loss_type == "dr_grpo":
        loss = (per_token * maskf).sum() / (mask.shape[0] * max_len)
    elif loss_type in ("dapo", "cispo", "vespo"):
        loss = (per_token * maskf).sum() / maskf.sum().clamp(min=1)
    elif loss_type == "luspo":
        loss = (per_token * maskf.sum(1, keepdim=True)).mean()
    loss.backward()
    return dict(loss=loss.detach(), gx=x.grad, gw=w.grad, logps=lp.detach())


def case(device, dtype, batch=4, seq=24, hidden=64, vocab=500, use_ref=True, with_old=True, **kw):
    from liger_kernel_b200 import chunked_loss as cl

    g = torch.Generator().manual_seed(batch * 31 + seq)
    x = torch.randn(batch, seq, hidden, generator=g).to(dtype)
    w = (torch.randn(vocab, hidden, generator=g) * 0.1).to(dtype)
    ids = torch.randint(0, vocab, (batch, seq), generator=g)
    mask = (torch.rand(batch, seq, generator=g) < 0.8).long()
    mask[:, 0] = 1
    adv = torch.randn(batch, generator=g)
    ref = ((torch.randn(batch, seq, hidden, generator=g)).to(dtype), (torch.randn(vocab, hidden, generator=g) * 0.1).to(dtype)) if use_ref else None
    temperature = kw.get("temperature", 1.0)
    old = None
    if with_old:      # sampled under a slightly different policy: ratios on both sides of the clip
        with torch.no_grad():
            lp = F.log_softmax((x.double() @ w.double().t()) / temperature, dim=-1)
            old = (torch.gather(lp, 2, ids.unsqueeze(2)).squeeze(2) + torch.randn(batch, seq, generator=g).double() * 0.3).float()
    want = torch_grpo(x, w, ids, mask, adv, ref=ref, old=old, beta=kw.get("beta", 0.04), eps_lo=kw.get("epsilon_low", 0.2),
                      eps_hi=kw.get("epsilon_high", 0.2), loss_type=kw.get("loss_type", "dapo"), max_len=kw.get("max_completion_length"),
                      level=kw.get("importance_sampling_level", "token"), temperature=temperature, delta=kw.get("delta"),
                      bias_corr=kw.get("use_bias_correction_kl", False))
    xd, wd = x.to(device).requires_grad_(True), w.to(device).requires_grad_(True)
    mod = cl.LigerFusedLinearGRPOLoss(use_ref_model=use_ref, **kw)
    loss, metrics = mod(xd, wd, ids.to(device), mask.to(device), adv.to(device), None, None, None if old is None else old.to(device),
                        None if ref is None else ref[0].to(device), None if ref is None else ref[1].to(device))
    low = dtype != torch.float32
    tol = 3e-2 if low else 3e-4
    assert_close(loss.detach().float().cpu().reshape(()), want["loss"].float(), tol * max(1.0, float(want["loss"].abs())), tol, "loss")
    assert len(metrics) == (2 if kw.get("beta", 0.04) != 0 else 1) and all(m.dim() == 0 for m in metrics)
    loss.backward()
    for name, got, ref_g in (("grad_input", xd.grad, want["gx"]), ("grad_weight", wd.grad, want["gw"])):
        ref_g = ref_g.float()
        assert got.dtype == dtype and got.shape == ref_g.shape
        assert_close(got.float().cpu(), ref_g, (3e-2 if low else 3e-5) * float(ref_g.abs().max()), 6e-2 if low else 3e-3, name)
    if kw.get("loss_type") != "luspo":
        assert float(xd.grad[mask.to(device) == 0].abs().max()) == 0.0    # positions outside the mask are not evaluated
