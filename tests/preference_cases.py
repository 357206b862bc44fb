"""Shared bodies of the preference-loss tests (DPO / ORPO / SimPO / CPO on the fused head): run on a B200
(tests/test_preference_losses_gpu.py) and with the kernels emulated on the host (tests/test_preference_losses_emulation_cpu.py).

The checker is torch in float64 with materialised logits, written the way the reference's own tests write theirs
(test/utils.py HFAlignmentLoss.get_batch_logps / concatenated_forward, test/chunked_loss/test_{dpo,orpo,simpo,cpo}_loss.py):
log_softmax over the vocabulary, gather at the labels, masked sum or mean per sequence, then the pairwise formula of each
paper, differentiated by autograd."""

import torch
import torch.nn.functional as F

from flce_cases import assert_close


def batch_logps(x, w, b, target, average, ignore_index=-100):
    logits = x @ w.t() + (0 if b is None else b)
    lp = F.log_softmax(logits, dim=-1)
    mask = target != ignore_index
    tok = torch.gather(lp, 2, torch.where(mask, target, 0).unsqueeze(2)).squeeze(2) * mask
    seq = tok.sum(-1)
    return (seq / mask.sum(-1) if average else seq), tok, mask, logits


def torch_reference(kind, x, w, b, target, ref=None, beta=0.1, alpha=1.0, compute_nll=True, average=True, **kw):
    x = x.double().requires_grad_(True)
    w = w.double().requires_grad_(True)
    b = None if b is None else b.double().requires_grad_(True)
    pairs = x.shape[0] // 2
    seq, tok, mask, logits = batch_logps(x, w, b, target, average)
    pc, pr = seq[:pairs], seq[pairs:]
    nll = -(tok[:pairs].sum()) / mask[:pairs].sum() if compute_nll else torch.zeros((), dtype=torch.float64)
    if kind == "dpo":
        rc = rr = 0.0
        if ref is not None:
            rseq = batch_logps(ref[0].double(), ref[1].double(), None, target, average)[0]
            rc, rr = rseq[:pairs], rseq[pairs:]
        margin = beta * ((pc - pr) - (rc - rr))
        lt = kw.get("loss_type", "sigmoid")
        ls = kw.get("label_smoothing", 0.0)
        if lt == "sigmoid":
            pref = -F.logsigmoid(margin).mean()
        elif lt == "hinge":
            pref = torch.relu(1 - margin).mean()
        elif lt == "robust":
            pref = ((-(1 - ls) * F.logsigmoid(margin) + ls * F.logsigmoid(-margin)) / (1 - 2 * ls)).mean()
        elif lt == "sppo_hard":
            pref = (((pc - rc) - 0.5 / beta) ** 2 + ((pr - rr) + 0.5 / beta) ** 2).mean()
        else:
            raise AssertionError(lt)
    elif kind == "orpo":
        log_odds = (pc - pr) - (torch.log1p(-torch.exp(pc)) - torch.log1p(-torch.exp(pr)))
        pref = -beta * F.logsigmoid(log_odds).mean()
    elif kind == "simpo":
        z = beta * (pc - pr) - kw.get("gamma", 0.5)
        ls = kw.get("label_smoothing", 0.0)
        pref = (-F.logsigmoid(z) * (1 - ls) - F.logsigmoid(-z) * ls).mean()
    elif kind == "cpo":
        z = beta * (pc - pr)
        ls = kw.get("label_smoothing", 0.0)
        pref = (-F.logsigmoid(z) * (1 - ls) - F.logsigmoid(-z) * ls).mean()
    loss = alpha * nll + pref
    loss.backward()
    return dict(loss=loss.detach(), chosen=pc.detach(), rejected=pr.detach(), nll=nll.detach(), gx=x.grad, gw=w.grad,
                gb=None if b is None else b.grad, chosen_logits_mean=logits[:pairs].mean().detach(),
                rejected_logits_mean=logits[pairs:].mean().detach())


def make_batch(pairs, seq, hidden, vocab, dtype, seed=0, with_bias=False):
    g = torch.Generator().manual_seed(seed + pairs * 7 + seq)
    x = (torch.randn(2 * pairs, seq, hidden, generator=g)).to(dtype)
    w = (torch.randn(vocab, hidden, generator=g) * 0.1).to(dtype)
    b = (torch.randn(vocab, generator=g) * 0.1).to(dtype) if with_bias else None
    t = torch.randint(0, vocab, (2 * pairs, seq), generator=g)
    t[:, : seq // 3] = -100                         # the prompt
    t[torch.rand(2 * pairs, seq, generator=g) < 0.1] = -100
    t[:, -1] = 1                                    # every sequence keeps at least one completion token
    return x, w, b, t


def check(out, want, dtype):
    loss, aux = out
    low = dtype != torch.float32
    tol = 2e-2 if low else 2e-4
    assert_close(loss.detach().float().cpu().reshape(()), want["loss"].float(), tol * max(1.0, float(want["loss"].abs())), tol, "loss")
    assert_close(aux[0].float().cpu(), want["chosen"].float(), tol * float(want["chosen"].abs().max()), tol, "chosen_logps")
    assert_close(aux[1].float().cpu(), want["rejected"].float(), tol * float(want["rejected"].abs().max()), tol, "rejected_logps")
    assert_close(aux[4].float().cpu().reshape(()), want["nll"].float(), tol * max(1.0, float(want["nll"])), tol, "nll")
    assert_close(aux[2].float().cpu().reshape(()), want["chosen_logits_mean"].float(), 2e-3, 5e-2, "chosen_logits_mean")
    assert_close(aux[3].float().cpu().reshape(()), want["rejected_logits_mean"].float(), 2e-3, 5e-2, "rejected_logits_mean")


def case(device, kind, dtype, pairs=3, seq=24, hidden=64, vocab=500, with_bias=False, use_ref=False, **kw):
    from liger_kernel_b200 import chunked_loss as cl

    x, w, b, t = make_batch(pairs, seq, hidden, vocab, dtype, with_bias=with_bias)
    ref = None
    if use_ref:
        rx, rw, _, _ = make_batch(pairs, seq, hidden, vocab, dtype, seed=99)
        ref = (rx, rw)
    beta = kw.pop("beta", 0.1)
    want = torch_reference(kind, x, w, b, t, ref=ref, beta=beta, **kw)
    xd = x.to(device).requires_grad_(True)
    wd = w.to(device).requires_grad_(True)
    bd = None if b is None else b.to(device).requires_grad_(True)
    td = t.to(device)
    compute_nll = kw.get("compute_nll", True)
    alpha = kw.get("alpha", 1.0)
    if kind == "dpo":
        mod = cl.LigerFusedLinearDPOLoss(beta=beta, alpha=alpha, compute_nll_loss=compute_nll, use_ref_model=use_ref,
                                         average_log_prob=kw.get("average", True), loss_type=kw.get("loss_type", "sigmoid"),
                                         label_smoothing=kw.get("label_smoothing", 0.0))
        out = mod(wd, xd, td, bd, None if ref is None else ref[0].to(device), None if ref is None else ref[1].to(device), None)
    elif kind == "orpo":
        out = cl.LigerFusedLinearORPOLoss(beta=beta, compute_nll_loss=compute_nll)(wd, xd, td, bd)
    elif kind == "simpo":
        out = cl.LigerFusedLinearSimPOLoss(beta=beta, alpha=alpha, compute_nll_loss=compute_nll, gamma=kw.get("gamma", 0.5),
                                           label_smoothing=kw.get("label_smoothing", 0.0))(wd, xd, td, bd)
    else:
        out = cl.LigerFusedLinearCPOLoss(beta=beta, alpha=alpha, compute_nll_loss=compute_nll,
                                         average_log_prob=kw.get("average", True),
                                         label_smoothing=kw.get("label_smoothing", 0.0))(wd, xd, td, bd)
    check(out, want, dtype)
    out[0].backward()
    low = dtype != torch.float32
    for name, got, ref_g in (("grad_input", xd.grad, want["gx"]), ("grad_weight", wd.grad, want["gw"]),
                             ("grad_bias", None if bd is None else bd.grad, want["gb"])):
        if ref_g is None:
            continue
        ref_g = ref_g.float()
        assert got.shape == ref_g.shape and got.dtype == dtype, name
        assert_close(got.float().cpu(), ref_g, (2e-2 if low else 2e-5) * float(ref_g.abs().max()), 5e-2 if low else 2e-3, name)
    # the prompt and the ignored positions take no part
    assert float(xd.grad[td == -100].abs().max()) == 0.0


def case_kto(device, dtype, batch=5, seq=20, hidden=64, vocab=300, use_ref=True, with_kl=True, average=False, beta=0.3):
    from liger_kernel_b200 import chunked_loss as cl

    x, w, _, t = make_batch((batch + 1) // 2, seq, hidden, vocab, dtype)
    x, t = x[:batch], t[:batch]
    labels = torch.tensor([i % 3 != 1 for i in range(batch)])
    g = torch.Generator().manual_seed(5)
    kl = torch.rand(batch, generator=g) * 0.5 if with_kl else None
    ref = make_batch((batch + 1) // 2, seq, hidden, vocab, dtype, seed=99)[:2] if use_ref else None
    # torch, float64, materialised logits
    xr, wr = x.double().requires_grad_(True), w.double().requires_grad_(True)
    seq_lp, _, _, logits = batch_logps(xr, wr, None, t, average)
    ratios = seq_lp
    if use_ref:
        ratios = seq_lp - batch_logps(ref[0][:batch].double(), ref[1].double(), None, t, average)[0]
    z = ratios - kl.double() if with_kl else ratios
    want = (1 - torch.sigmoid(beta * z * torch.where(labels, 1.0, -1.0))).mean()
    want.backward()
    xd, wd = x.to(device).requires_grad_(True), w.to(device).requires_grad_(True)
    mod = cl.LigerFusedLinearKTOLoss(beta=beta, use_ref_model=use_ref, average_log_prob=average)
    loss, aux = mod(xd, wd, t.to(device), None, labels.to(device), None if ref is None else ref[0][:batch].to(device),
                    None if ref is None else ref[1].to(device), None, None if kl is None else kl.to(device))
    low = dtype != torch.float32
    tol = 2e-2 if low else 2e-4
    assert_close(loss.detach().float().cpu().reshape(()), want.detach().float(), tol, tol, "loss")
    assert_close(aux[0].float().cpu().reshape(()), (seq_lp.detach() * labels).sum().float(), tol * float(seq_lp.detach().abs().sum()), tol,
                 "chosen_logps_sum")
    assert_close(aux[2].float().cpu().reshape(()), (logits.detach().sum((1, 2)) * labels).sum().float(),
                 2e-2 * float(logits.detach().abs().sum()) ** 0.5 + 1.0, 5e-2, "chosen_logits_sum")
    loss.backward()
    for name, got, ref_g in (("grad_input", xd.grad, xr.grad), ("grad_weight", wd.grad, wr.grad)):
        ref_g = ref_g.float()
        assert_close(got.float().cpu(), ref_g, (2e-2 if low else 2e-5) * float(ref_g.abs().max()), 5e-2 if low else 2e-3, name)
