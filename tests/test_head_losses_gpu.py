"""Fused linear JSD and fused linear scaled cross-entropy on a B200 against the CPU oracle and the reference's golden
vectors.  Case grids follow test/transformers/test_fused_linear_jsd.py and test_fused_linear_scaled_cross_entropy.py of
the reference (shapes with odd sizes and a 128 k-wide vocabulary, dtypes, beta 0 / 1 / in between, temperatures, labels
with ignore_index, upstream gradients, single-output backward).

The case bodies live in tests/head_loss_cases.py; tests/test_head_losses_emulation_cpu.py runs the same bodies on CPU
tensors with the row kernels emulated on the host."""

import pytest
import torch

import head_loss_cases as cases
from golden_util import jsd_golden_names, sce_golden_names

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,Hs,Ht,V", [(512, 256, 512, 4096), (141, 31, 57, 1423), (256, 128, 256, 128256)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("beta,temperature,labels", [(0.5, 1.0, None), (0.1, 2.0, 0.2), (0.0, 1.0, 0.2), (1.0, 0.5, None)])
def test_jsd_correctness(N, Hs, Ht, V, dtype, beta, temperature, labels):
    if V > 100000 and dtype == torch.float32 and beta != 0.5:
        pytest.skip("one fp32 case at the wide vocabulary is enough")
    cases.case_jsd_correctness("cuda", N, Hs, Ht, V, dtype, beta, temperature, labels)


def test_jsd_functional_upstream_gradient_and_ignore_index():
    cases.case_jsd_correctness("cuda", 300, 64, 128, 1000, torch.bfloat16, 0.5, 1.0, 0.1, grad_output=2.5, functional=True)
    cases.case_jsd_correctness("cuda", 300, 64, 128, 1000, torch.float32, 0.7, 1.5, 0.3, ignore_index=7, grad_output=0.5)


@pytest.mark.parametrize("name", jsd_golden_names())
def test_jsd_against_reference_golden(name):
    cases.case_jsd_golden("cuda", name)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_jsd_multichunk(dtype):
    cases.case_jsd_multichunk_equals_single_chunk("cuda", dtype)


def test_jsd_all_ignored():
    cases.case_jsd_all_ignored("cuda")


def test_jsd_weight_without_grad_and_second_backward():
    cases.case_jsd_weight_without_grad_and_second_backward("cuda")


@pytest.mark.parametrize("N,H,V,dtype", [(17, 31, 257, torch.float32), (1025, 64, 131072, torch.bfloat16), (512, 256, 4096, torch.float16),
                                         (300, 128, 32001, torch.float32)])
@pytest.mark.parametrize("temperature,grads", [(1.0, "both"), (1.5, "nll"), (0.7, "entropy")])
@pytest.mark.parametrize("mode", ["fused", "chunked"])
def test_scaled_ce_correctness(N, H, V, dtype, temperature, grads, mode):
    if mode == "fused" and dtype == torch.float32:
        pytest.skip("fp32 operands always take the chunked form")
    cases.case_sce_correctness("cuda", N, H, V, dtype, temperature, grads, mode=mode)


@pytest.mark.parametrize("mode", ["fused", "chunked"])
@pytest.mark.parametrize("name", sce_golden_names())
def test_scaled_ce_against_reference_golden(name, mode):
    cases.case_sce_golden("cuda", name, mode=mode)


def test_scaled_ce_fused_several_gradient_slabs(monkeypatch):
    """A slab budget that cuts the vocabulary into several logit-gradient slabs (fp32 accumulation of grad_input across them)."""
    import liger_kernel_b200.ops.fused_linear_scaled_cross_entropy as mod

    monkeypatch.setattr(mod, "SLAB_BUDGET_BYTES", 300 * 512 * 2)            # 512 classes per slab for 300 rows
    cases.case_sce_correctness("cuda", 300, 72, 2000, torch.bfloat16, 1.3, "both", mode="fused")


def test_scaled_ce_multichunk_single_output_and_errors(monkeypatch):
    import liger_kernel_b200.ops._chunked as ck

    monkeypatch.setattr(ck, "SLAB_BUDGET_BYTES", 256 * ck.slab_pitch(67) * 2)          # 256 rows per chunk
    cases.case_sce_correctness("cuda", 600, 16, 67, torch.bfloat16, 1.25, "both", mode="chunked")
    cases.case_sce_nll_only_output_and_no_grad("cuda")
    cases.case_sce_argument_errors("cuda")
