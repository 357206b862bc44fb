"""Stand-alone cross-entropy on materialised logits (LigerCrossEntropyFunction) against the CPU oracle and the
reference's golden vectors.  Case grid follows test/transformers/test_cross_entropy.py of the reference
(shapes incl. V=128256-like wide rows and odd sizes, dtypes, reductions, label smoothing, z-loss, soft-cap,
class weights, ignore_index, not-last-layer upstream gradients, per-row gradients for reduction "none").

The case bodies live in tests/ce_cases.py; tests/test_simt_emulation_cpu.py runs the same bodies on CPU tensors with
the kernels emulated on the host."""

import pytest
import torch

import ce_cases
from golden_util import ce_golden_names

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,V", [(256, 4096), (188, 123), (64, 128256), (33, 32001)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("reduction", ["mean", "sum"])
@pytest.mark.parametrize("feat", ce_cases.FEATURES)
def test_ce_correctness(N, V, dtype, reduction, feat):
    ce_cases.case_correctness("cuda", N, V, dtype, reduction, feat)


def test_ce_weights_none_reduction_upstream_gradient_and_inplace():
    ce_cases.case_weights_none_reduction_upstream_gradient_and_inplace("cuda")


def test_ce_all_ignored_is_exact_zero():
    ce_cases.case_all_ignored_is_exact_zero("cuda")


@pytest.mark.parametrize("name", ce_golden_names())
def test_ce_against_reference_golden(name):
    ce_cases.case_reference_golden("cuda", name)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("label_smoothing", [0.0, 0.1])
@pytest.mark.parametrize("reduction", ["sum", "mean"])
def test_ce_true_class_gradient_confident_predictions(dtype, label_smoothing, reduction):
    ce_cases.case_true_class_gradient_confident_predictions("cuda", dtype, label_smoothing, reduction)


def test_ce_forward_only_structured_output_and_target_check():
    ce_cases.case_forward_only_structured_output_and_target_check("cuda")
