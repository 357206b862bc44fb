"""Shared bodies of the tests of the fused RMSNorm + lm_head + cross-entropy operator: run on a B200
(tests/test_rmsnorm_head_gpu.py) and, with the row kernels emulated on the host, on CPU tensors
(tests/test_rmsnorm_head_emulation_cpu.py).

The checker is torch in float64 on the host: the reference's RMSNorm formula (src/liger_kernel/ops/rms_norm.py:59-139; test
pattern of test/transformers/test_rms_norm.py: LlamaRMSNorm / GemmaRMSNorm in torch against the kernel) feeding a linear layer
and torch's cross-entropy, differentiated by autograd."""

import torch
import torch.nn.functional as F

from flce_cases import assert_close


def reference(hidden, gamma, weight, target, eps, offset, casting_mode, dtype, reduction="mean", ignore_index=-100,
              label_smoothing=0.0, grad_output=1.0):
    h = hidden.to(dtype).double().requires_grad_(True)
    g = gamma.to(dtype).double().requires_grad_(True)
    w = weight.to(dtype).double().requires_grad_(True)
    rstd = torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    y = h * rstd * (offset + g)
    logits = y @ w.t()
    loss = F.cross_entropy(logits, target, ignore_index=ignore_index, label_smoothing=label_smoothing, reduction=reduction)
    (loss * grad_output).backward()
    # what the tensor cores are fed: the normalised rows rounded to the input dtype (per casting mode)
    with torch.no_grad():
        hf = hidden.to(dtype).float()
        r = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
        if casting_mode == "llama":
            normed = ((hf * r).to(dtype).float() * (offset + gamma.to(dtype).float())).to(dtype)
        else:
            normed = (hf * r * (offset + gamma.to(dtype).float())).to(dtype)
    return dict(loss=loss.detach(), grad_hidden=h.grad, grad_gamma=g.grad, grad_weight=w.grad, normed=normed)


def make_case(n, hidden, vocab, ignored, seed=0):
    g = torch.Generator().manual_seed(seed + n + hidden)
    h = torch.randn(n, hidden, generator=g) * 3.0 + 0.2
    gamma = torch.rand(hidden, generator=g) + 0.5
    w = torch.randn(vocab, hidden, generator=g) * 0.05
    t = torch.randint(0, vocab, (n,), generator=g)
    t[torch.rand(n, generator=g) < ignored] = -100
    if ignored > 0:
        t[0] = -100
    return h, gamma, w, t


def case_matches_torch(device, n, hidden, vocab, dtype, casting_mode, offset, reduction="mean", label_smoothing=0.0,
                       ignored=0.2, grad_output=1.0):
    import liger_kernel_b200 as lk

    eps = 1e-6
    h, gamma, w, t = make_case(n, hidden, vocab, ignored)
    ref = reference(h, gamma, w, t, eps, offset, casting_mode, dtype, reduction, label_smoothing=label_smoothing,
                    grad_output=grad_output)
    hd = h.to(dtype).to(device).requires_grad_(True)
    gd = gamma.to(dtype).to(device).requires_grad_(True)
    wd = w.to(dtype).to(device).requires_grad_(True)
    loss = lk.liger_fused_rmsnorm_linear_cross_entropy(hd, gd, wd, t.to(device), eps=eps, offset=offset,
                                                       casting_mode=casting_mode, reduction=reduction,
                                                       label_smoothing=label_smoothing)
    (loss * grad_output).backward()
    scale = max(1.0, float(ref["loss"].abs()))
    assert_close(loss.detach().float().cpu(), ref["loss"].float(), 2e-2 * scale, 2e-2, "loss")
    for name, got, want in (("grad_hidden", hd.grad, ref["grad_hidden"]), ("grad_gamma", gd.grad, ref["grad_gamma"]),
                            ("grad_weight", wd.grad, ref["grad_weight"])):
        want = want.float()
        assert got.dtype == dtype and got.shape == want.shape, name
        assert_close(got.float().cpu(), want, 2e-2 * float(want.abs().max()), 5e-2, name)
    # ignored tokens: exact zeros
    assert float(hd.grad[t.to(device) == -100].abs().max()) == 0.0 if ignored > 0 else True
    # the unfused composition through the library's own head gives the same loss on the same rounded rows
    plain = lk.liger_fused_linear_cross_entropy(ref["normed"].to(device), wd.detach(), t.to(device), reduction=reduction,
                                                label_smoothing=label_smoothing)
    assert_close(loss.detach().float().cpu(), plain.float().cpu(), 2e-3 * scale, 2e-3, "loss vs unfused composition")


def case_forward_only_and_rejections(device):
    import pytest

    import liger_kernel_b200 as lk

    h, gamma, w, t = make_case(40, 64, 300, 0.2)
    dtype = torch.bfloat16
    ref = reference(h, gamma, w, t, 1e-6, 0.0, "llama", dtype)
    args = (h.to(dtype).to(device), gamma.to(dtype).to(device), w.to(dtype).to(device), t.to(device))
    with torch.no_grad():
        loss = lk.liger_fused_rmsnorm_linear_cross_entropy(*args)
    assert_close(loss.float().cpu(), ref["loss"].float(), 2e-2, 2e-2, "loss (no grad)")
    out = lk.liger_fused_rmsnorm_linear_cross_entropy(*args, return_token_accuracy=True, return_predicted_tokens=True)
    assert isinstance(out, lk.CrossEntropyOutput) and out.predicted_tokens.shape == (40,)
    assert torch.all(out.predicted_tokens[t.to(device) == -100] == -1)
    hg = args[0].clone().requires_grad_(True)
    with pytest.raises(NotImplementedError, match="reduction"):
        lk.liger_fused_rmsnorm_linear_cross_entropy(hg, *args[1:], reduction="none")
    with pytest.raises(NotImplementedError, match="casting_mode"):
        lk.liger_fused_rmsnorm_linear_cross_entropy(hg, *args[1:], casting_mode="none")
    with pytest.raises(NotImplementedError, match="multiple of 8"):
        lk.liger_fused_rmsnorm_linear_cross_entropy(hg[:, :60].contiguous(), args[1][:60].contiguous(), args[2][:, :60].contiguous(),
                                                    args[3])
    loss = lk.liger_fused_rmsnorm_linear_cross_entropy(hg, *args[1:])
    loss.backward(retain_graph=True)
    with pytest.raises(RuntimeError, match="handed out once"):
        loss.backward()
