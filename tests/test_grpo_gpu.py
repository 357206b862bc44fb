"""GRPO on the fused head on a B200 against torch in float64 with materialised logits (body in tests/grpo_cases.py)."""

import pytest
import torch

import grpo_cases as cases
from test_grpo_emulation_cpu import VARIANTS

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kw", VARIANTS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_grpo(kw, dtype):
    cases.case("cuda", dtype, batch=4, seq=48, hidden=256, vocab=4099, **dict(kw))


def test_on_policy_wide_vocabulary():
    cases.case("cuda", torch.bfloat16, batch=2, seq=64, hidden=512, vocab=32001, use_ref=False, with_old=False, loss_type="grpo")
