"""CPU stand-in for the local FLCE pieces, used only to exercise the cross-rank exchange logic of
liger_kernel_b200.sharded on gloo ranks.  It produces the same intermediate quantities as the CUDA library
(normalisers, [6, N] row statistics, per-row outputs, shard-local gradients) with plain torch fp64 math."""

from types import SimpleNamespace

import torch


class CpuBackend:
    def prepare(self, x, w, target, bias, ce_weight, ignore_index, lse_square_scale, label_smoothing, reduction, softcap,
                use_token_scaling, vocab_total=None, vocab_offset=0, want_argmax=False):
        assert bias is None and ce_weight is None and not use_token_scaling
        return SimpleNamespace(
            x=x.double(), w=w.double(), target=target.long(), ignore_index=ignore_index, lam=lse_square_scale,
            alpha=label_smoothing, reduction=reduction, softcap=softcap, vocab_total=vocab_total or w.shape[0],
            vocab_offset=vocab_offset, device=x.device, n_rows=x.shape[0], hidden=x.shape[1], vocab=w.shape[0], dtype=x.dtype)

    def count(self, p):
        n = float((p.target != p.ignore_index).sum())
        return torch.tensor([n, n, float(p.vocab_total), 0.0], dtype=torch.float32)

    def _logits(self, p):
        z = p.x @ p.w.t()
        return z if p.softcap is None else p.softcap * torch.tanh(z / p.softcap)

    def forward_stats(self, p):
        s = self._logits(p)
        m = s.max(dim=1).values
        d = torch.exp(s - m[:, None]).sum(dim=1)
        local = p.target - p.vocab_offset
        own = (local >= 0) & (local < p.vocab)
        xy = torch.where(own, s.gather(1, local.clamp(0, p.vocab - 1)[:, None])[:, 0], torch.zeros_like(m))
        best_val, best_idx = s.max(dim=1)
        idx_bits = (best_idx + p.vocab_offset).to(torch.int32).view(torch.float32)
        return torch.stack([m.float(), d.float(), xy.float(), s.sum(dim=1).float(), best_val.float(), idx_bits], dim=0)

    def finalize(self, p, rowstats, norm):
        m, d, xy, ss = (rowstats[i].double() for i in range(4))
        amax = rowstats[5].contiguous().view(torch.int32).long()
        valid = p.target != p.ignore_index
        lse = m + torch.log(d)
        eps = p.alpha / p.vocab_total
        loss = lse - xy
        if p.alpha > 0:
            loss = loss * (1 - p.alpha) + (-eps * ss + p.alpha * lse)
        z = p.lam * lse * lse
        if p.reduction == "mean":
            loss, z = loss / float(norm[1]), z / float(norm[0])
        loss = torch.where(valid, loss + z, torch.zeros_like(loss))
        z = torch.where(valid, z, torch.zeros_like(z))
        pred = torch.where(valid, amax, torch.full_like(amax, -1))
        correct = ((amax == p.target) & valid).float()
        scalars = torch.stack([loss.sum(), z.sum(), correct.sum() / float(norm[0]), norm[0].double()]).float()
        return dict(lse=lse.float(), target_prob=torch.exp(xy - lse).float(), loss_rows=loss.float(), z_loss_rows=z.float(),
                    correct_rows=correct, predicted_tokens=pred, scalars=scalars)

    def backward(self, p, lse, target_prob, norm, grad_output, need_input, need_weight, grad_dtype=None, slab_hook=None):
        s = self._logits(p)
        prob = torch.exp(s - lse.double()[:, None])
        valid = (p.target != p.ignore_index).double()
        go = torch.ones(p.n_rows, dtype=torch.float64) if grad_output is None else grad_output.double().reshape(-1).expand(p.n_rows)
        inv_n = 1.0 / float(norm[0]) if p.reduction == "mean" else 1.0
        base = go * valid * inv_n
        eps = p.alpha / p.vocab_total
        g = prob * (base * (1 + 2 * p.lam * lse.double()))[:, None] - (base * eps)[:, None]
        local = p.target - p.vocab_offset
        own = (local >= 0) & (local < p.vocab)
        rows = torch.arange(p.n_rows)[own]
        g[rows, local[own]] -= (base * (1 - p.alpha))[own]
        if p.softcap is not None:
            g = g * (1 - (s / p.softcap) ** 2)
        gx = (g @ p.w).float() if need_input else None
        gw = (g.t() @ p.x).float() if need_weight else None
        if slab_hook is not None and gw is not None:
            slab_hook(0, p.vocab, gw)
        return gx, gw
