"""JSD distillation (hard CE + soft generalised JSD) on the fused operators on a B200 against torch in float64."""

import pytest
import torch

import distillation_cases as cases
from test_distillation_emulation_cpu import VARIANTS

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kw", VARIANTS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_jsd_distillation(kw, dtype):
    cases.case("cuda", dtype, rows=300, hs=256, ht=384, vocab=4099, **dict(kw))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("kw", [dict(), dict(wh=0.0, wsft=1.0, beta=1.0), dict(wh=1.0, wsft=0.3, beta=0.7)])
def test_cosine_similarity_distillation(kw, dtype):
    cases.case_cosine("cuda", dtype, rows=300, hs=256, ht=384, vocab=40000, **dict(kw))
