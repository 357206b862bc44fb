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
