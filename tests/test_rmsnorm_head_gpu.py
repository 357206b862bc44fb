"""Fused RMSNorm + lm_head + cross-entropy on a B200 against torch in float64 (bodies in tests/rmsnorm_head_cases.py)."""

import pytest
import torch

import rmsnorm_head_cases as cases

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,hidden,vocab", [(300, 256, 1000), (1000, 4096, 4099), (77, 8192, 515), (130, 16384, 260), (64, 72, 333)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("casting_mode,offset", [("llama", 0.0), ("gemma", 1.0)])
def test_matches_torch(n, hidden, vocab, dtype, casting_mode, offset):
    cases.case_matches_torch("cuda", n, hidden, vocab, dtype, casting_mode, offset)


@pytest.mark.parametrize("reduction,label_smoothing,ignored,grad_output", [("sum", 0.0, 0.2, 1.0), ("mean", 0.1, 0.0, 0.5),
                                                                          ("mean", 0.0, 0.9, 2.0)])
def test_reductions_smoothing_upstream_gradient(reduction, label_smoothing, ignored, grad_output):
    cases.case_matches_torch("cuda", 500, 1024, 2000, torch.bfloat16, "llama", 0.0, reduction, label_smoothing, ignored, grad_output)


def test_forward_only_and_rejections():
    cases.case_forward_only_and_rejections("cuda")
