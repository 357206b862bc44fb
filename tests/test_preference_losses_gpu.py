"""DPO / ORPO / SimPO / CPO on the fused head on a B200 against torch in float64 with materialised logits
(bodies in tests/preference_cases.py)."""

import pytest
import torch

import preference_cases as cases

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind,kw", [
    ("dpo", dict(use_ref=True, average=False, compute_nll=False)),
    ("dpo", dict(use_ref=False, loss_type="hinge", compute_nll=True, alpha=0.5)),
    ("dpo", dict(use_ref=True, loss_type="robust", label_smoothing=0.1, beta=0.5)),
    ("dpo", dict(use_ref=True, loss_type="sppo_hard", average=True, compute_nll=False)),
    ("orpo", dict()),
    ("simpo", dict(gamma=0.3, label_smoothing=0.1, compute_nll=False)),
    ("cpo", dict(average=False, alpha=0.7)),
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_preference_loss(kind, kw, dtype):
    cases.case("cuda", kind, dtype, pairs=3, seq=40, hidden=256, vocab=4099, **dict(kw))


def test_with_bias_and_a_wide_vocabulary():
    cases.case("cuda", "orpo", torch.bfloat16, pairs=2, seq=64, hidden=512, vocab=32001, with_bias=True)
    cases.case("cuda", "dpo", torch.bfloat16, pairs=2, seq=64, hidden=512, vocab=32001, use_ref=True, average=False,
               compute_nll=False)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("use_ref,with_kl,average", [(True, True, False), (False, False, True)])
def test_kto(dtype, use_ref, with_kl, average):
    cases.case_kto("cuda", dtype, batch=7, seq=48, hidden=256, vocab=4099, use_ref=use_ref, with_kl=with_kl, average=average)
