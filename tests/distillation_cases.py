"""Shared body of the JSD-distillation tests: the library's operator against torch in float64 with materialised logits, written
as the reference's test writes its checker (test/chunked_loss/test_jsd_loss.py: HFJSDLoss on HFDistillationLoss)."""

import math

import torch
import torch.nn.functional as F

from flce_cases import assert_close


def torch_distillation(xs, ws, xt, wt, labels, wh, wsft, beta, temperature, ignore_index=-100):
    xs = xs.double().requires_grad_(True)
    ws = ws.double().requires_grad_(True)
    s_logits = xs @ ws.t()
    t_logits = xt.double() @ wt.double().t()
    n = (labels != ignore_index).sum().clamp_min(1)
    hard = F.cross_entropy(s_logits, labels, ignore_index=ignore_index, reduction="sum") / n
    ls, lt = F.log_softmax(s_logits / temperature, -1), F.log_softmax(t_logits / temperature, -1)
    if beta == 0:
        rows = F.kl_div(ls, lt, reduction="none", log_target=True).sum(-1)
    elif beta == 1:
        rows = F.kl_div(lt, ls, reduction="none", log_target=True).sum(-1)
    else:
        lm = torch.logsumexp(torch.stack([ls + math.log(1 - beta), lt + math.log(beta)]), dim=0)
        rows = (beta * F.kl_div(lm, lt, reduction="none", log_target=True) + (1 - beta) * F.kl_div(lm, ls, reduction="none", log_target=True)).sum(-1)
    soft = rows.masked_fill(labels == ignore_index, 0.0).sum() / n
    loss = wh * hard + wsft * soft
    loss.backward()
    return dict(loss=loss.detach(), soft=soft.detach(), hard=hard.detach(), gx=xs.grad, gw=ws.grad)


def case(device, dtype, rows=60, hs=64, ht=96, vocab=500, wh=0.5, wsft=0.5, beta=0.5, temperature=1.0):
    from liger_kernel_b200 import chunked_loss as cl

    g = torch.Generator().manual_seed(rows + vocab)
    xs, xt = torch.randn(rows, hs, generator=g).to(dtype), torch.randn(rows, ht, generator=g).to(dtype)
    ws, wt = (torch.randn(vocab, hs, generator=g) * 0.1).to(dtype), (torch.randn(vocab, ht, generator=g) * 0.1).to(dtype)
    labels = torch.randint(0, vocab, (rows,), generator=g)
    labels[torch.rand(rows, generator=g) < 0.2] = -100
    want = torch_distillation(xs, ws, xt, wt, labels, wh, wsft, beta, temperature)
    xd, wd = xs.to(device).requires_grad_(True), ws.to(device).requires_grad_(True)
    mod = cl.LigerFusedLinearJSDLoss(weight_hard_loss=wh, weight_soft_loss=wsft, beta=beta, temperature=temperature,
                                     return_soft_hard_loss=True)
    loss, soft, hard = mod(xd, wd, xt.to(device), wt.to(device), labels.to(device))
    low = dtype != torch.float32
    tol = 2e-2 if low else 3e-4
    for name, got, ref in (("loss", loss, want["loss"]), ("soft", soft, want["soft"]), ("hard", hard, want["hard"])):
        assert_close(got.detach().float().cpu().reshape(()), ref.float(), tol * max(1.0, float(ref.abs())), tol, name)
    loss.backward()
    for name, got, ref in (("grad_input", xd.grad, want["gx"]), ("grad_weight", wd.grad, want["gw"])):
        ref = ref.float()
        assert got.dtype == dtype and got.shape == ref.shape
        assert_close(got.float().cpu(), ref, (3e-2 if low else 3e-5) * float(ref.abs().max()), 6e-2 if low else 3e-3, name)


def case_cosine(device, dtype, rows=60, hs=64, ht=96, vocab=500, wh=0.5, wsft=0.5, beta=0.5):
    from liger_kernel_b200 import chunked_loss as cl

    g = torch.Generator().manual_seed(rows + vocab + 1)
    xs, xt = torch.randn(rows, hs, generator=g).to(dtype), torch.randn(rows, ht, generator=g).to(dtype)
    ws, wt = (torch.randn(vocab, hs, generator=g) * 0.1).to(dtype), (torch.randn(vocab, ht, generator=g) * 0.1).to(dtype)
    wt[:, :hs] += ws.float().to(dtype)[:, : min(hs, ht)] * 2            # correlated heads: cosines away from zero
    labels = torch.randint(0, vocab, (rows,), generator=g)
    labels[torch.rand(rows, generator=g) < 0.2] = -100
    a = xs.double().requires_grad_(True)
    b = ws.double().requires_grad_(True)
    s_logits, t_logits = a @ b.t(), xt.double() @ wt.double().t()
    n = (labels != -100).sum().clamp_min(1)
    hard = F.cross_entropy(s_logits, labels, ignore_index=-100, reduction="sum") / n
    soft = (beta * (1 - F.cosine_similarity(F.normalize(s_logits, dim=-1), F.normalize(t_logits, dim=-1), dim=-1))).sum() / n
    want = wh * hard + wsft * soft
    want.backward()
    xd, wd = xs.to(device).requires_grad_(True), ws.to(device).requires_grad_(True)
    mod = cl.LigerFusedLinearCosineSimilarityLoss(weight_hard_loss=wh, weight_soft_loss=wsft, beta=beta, return_soft_hard_loss=True)
    loss, soft_got, hard_got = mod(xd, wd, xt.to(device), wt.to(device), labels.to(device))
    low = dtype != torch.float32
    tol = 2e-2 if low else 3e-4
    for name, got, ref in (("loss", loss, want), ("soft", soft_got, soft), ("hard", hard_got, hard)):
        assert_close(got.detach().float().cpu().reshape(()), ref.detach().float(), tol * max(1.0, float(ref.detach().abs())), tol, name)
    loss.backward()
    for name, got, ref in (("grad_input", xd.grad, a.grad), ("grad_weight", wd.grad, b.grad)):
        ref = ref.float()
        assert got.dtype == dtype and got.shape == ref.shape
        assert_close(got.float().cpu(), ref, (3e-2 if low else 3e-5) * float(ref.abs().max()), 6e-2 if low else 3e-3, name)
