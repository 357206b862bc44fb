"""GRPO on the fused head with the library's kernels emulated on the host, against torch in float64 with materialised
logits (body in tests/grpo_cases.py)."""

import pytest
import torch

import emu_lib
import grpo_cases as cases

VARIANTS = [
    dict(loss_type="dapo"),
    dict(loss_type="grpo", beta=0.1, use_bias_correction_kl=True),
    dict(loss_type="bnpo", beta=0.0, delta=1.1),
    dict(loss_type="dr_grpo", max_completion_length=30, importance_sampling_level="sequence"),
    dict(loss_type="cispo", epsilon_high=1.2),
    dict(loss_type="luspo", temperature=0.7),
    dict(loss_type="vespo", beta=0.02),
]


@pytest.mark.parametrize("kw", VARIANTS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_grpo(monkeypatch, kw, dtype):
    with emu_lib.installed(monkeypatch):
        cases.case("cpu", dtype, batch=3, seq=10, hidden=32, vocab=131, **dict(kw))


def test_on_policy_without_reference_and_rejections(monkeypatch):
    from liger_kernel_b200 import chunked_loss as cl

    with emu_lib.installed(monkeypatch):
        cases.case("cpu", torch.bfloat16, batch=2, seq=8, hidden=32, vocab=131, use_ref=False, with_old=False, loss_type="grpo")
        x = torch.randn(2, 4, 32).bfloat16()
        w = torch.randn(50, 32).bfloat16()
        ids, mask, adv = torch.zeros(2, 4, dtype=torch.long), torch.ones(2, 4, dtype=torch.long), torch.ones(2)
        with pytest.raises(ValueError, match="Unknown loss type"):
            cl.LigerFusedLinearGRPOLoss(use_ref_model=False, loss_type="nope")(x, w, ids, mask, adv)
        with pytest.raises(ValueError, match="Sequence-level"):
            cl.LigerFusedLinearGRPOLoss(use_ref_model=False, loss_type="cispo", importance_sampling_level="sequence")(x, w, ids, mask, adv)
        with pytest.raises(AssertionError, match="ref_per_token_logps or ref_input"):
            cl.LigerFusedLinearGRPOLoss(use_ref_model=True)(x, w, ids, mask, adv)
        with pytest.raises(ValueError, match="delta must be positive"):
            cl.LigerFusedLinearGRPOLoss(delta=0.0)
