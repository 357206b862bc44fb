"""Fused RMSNorm + lm_head + cross-entropy with the library's row kernels (the normalising gather, the backward scatter)
and register epilogues emulated on the host, through the Python operator, against torch in float64."""

import pytest
import torch

import emu_lib
import rmsnorm_head_cases as cases


@pytest.mark.parametrize("n,hidden,vocab", [(37, 64, 300), (20, 520, 131)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("casting_mode,offset", [("llama", 0.0), ("gemma", 1.0)])
def test_matches_torch(monkeypatch, n, hidden, vocab, dtype, casting_mode, offset):
    with emu_lib.installed(monkeypatch):
        cases.case_matches_torch("cpu", n, hidden, vocab, dtype, casting_mode, offset)


def test_sum_smoothing_upstream_gradient(monkeypatch):
    with emu_lib.installed(monkeypatch):
        cases.case_matches_torch("cpu", 30, 72, 200, torch.bfloat16, "llama", 0.0, "sum", 0.1, 0.3, 0.5)


def test_forward_only_and_rejections(monkeypatch):
    with emu_lib.installed(monkeypatch):
        cases.case_forward_only_and_rejections("cpu")
