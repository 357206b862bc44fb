"""DPO / ORPO / SimPO / CPO on the fused head with the library's kernels emulated on the host, against torch in float64
with materialised logits (bodies in tests/preference_cases.py)."""

import pytest
import torch

import emu_lib
import preference_cases as cases


@pytest.mark.parametrize("kind,kw", [
    ("dpo", dict(use_ref=True, average=False, compute_nll=False)),
    ("dpo", dict(use_ref=False, loss_type="hinge", compute_nll=True, alpha=0.5)),
    ("dpo", dict(use_ref=True, loss_type="robust", label_smoothing=0.1, beta=0.5)),
    ("dpo", dict(use_ref=True, loss_type="sppo_hard", average=True, compute_nll=False)),
    ("orpo", dict()),
    ("simpo", dict(gamma=0.3, label_smoothing=0.1, compute_nll=False)),
    ("cpo", dict(average=False, alpha=0.7)),
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_preference_loss(monkeypatch, kind, kw, dtype):
    with emu_lib.installed(monkeypatch):
        cases.case("cpu", kind, dtype, pairs=2, seq=12, hidden=32, vocab=131, **dict(kw))


def test_with_bias_and_rejections(monkeypatch):
    from liger_kernel_b200 import chunked_loss as cl

    with emu_lib.installed(monkeypatch):
        cases.case("cpu", "cpo", torch.bfloat16, pairs=2, seq=10, hidden=32, vocab=131, with_bias=True)
        x, w, _, t = cases.make_batch(2, 8, 32, 131, torch.bfloat16)
        with pytest.raises(ValueError, match="even"):
            cl.liger_fused_linear_orpo(x[:3], w, t[:3])
        with pytest.raises(ValueError, match="Unsupported loss_type"):
            cl.LigerFusedLinearDPOLoss(loss_type="nope")
        with pytest.raises(NotImplementedError, match="ipo"):
            cl.liger_fused_linear_dpo(x, w, t, None, None, None, None, -100, 0.1, False, True, False, False, 1, "ipo")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("use_ref,with_kl,average", [(True, True, False), (False, False, True)])
def test_kto(monkeypatch, dtype, use_ref, with_kl, average):
    with emu_lib.installed(monkeypatch):
        cases.case_kto("cpu", dtype, batch=5, seq=10, hidden=32, vocab=131, use_ref=use_ref, with_kl=with_kl, average=average)
