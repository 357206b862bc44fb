"""JSD distillation (hard CE + soft generalised JSD) on the fused operators with the kernels emulated on the host."""

import pytest
import torch

import distillation_cases as cases
import emu_lib

VARIANTS = [dict(), dict(beta=0.0, wh=0.0, wsft=1.0), dict(beta=1.0, temperature=2.0), dict(beta=0.3, wh=1.0, wsft=0.25, temperature=0.7)]


@pytest.mark.parametrize("kw", VARIANTS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_jsd_distillation(monkeypatch, kw, dtype):
    with emu_lib.installed(monkeypatch):
        cases.case("cpu", dtype, rows=24, hs=32, ht=48, vocab=131, **dict(kw))


def test_rejections(monkeypatch):
    from liger_kernel_b200 import chunked_loss as cl

    with emu_lib.installed(monkeypatch):
        x, w = torch.randn(4, 32).bfloat16(), torch.randn(50, 32).bfloat16()
        t = torch.zeros(4, dtype=torch.long)
        with pytest.raises(NotImplementedError, match="biases"):
            cl.liger_fused_linear_jsd(x, w, x, w, t, torch.zeros(50), None)
        with pytest.raises(NotImplementedError, match="vocabulary"):
            cl.liger_fused_linear_jsd(x, w, x, w[:40], t)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("kw", [dict(), dict(wh=0.0, wsft=1.0, beta=1.0), dict(wh=1.0, wsft=0.3, beta=0.7)])
def test_cosine_similarity_distillation(monkeypatch, kw, dtype):
    with emu_lib.installed(monkeypatch):
        cases.case_cosine("cpu", dtype, rows=24, hs=32, ht=48, vocab=131, **dict(kw))
