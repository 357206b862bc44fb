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
@pytest.mark.parametrize("mode", ["auto", "two_pass"])
def test_ce_correctness(N, V, dtype, reduction, feat, mode):
    ce_cases.case_correctness("cuda", N, V, dtype, reduction, feat, mode=mode)


@pytest.mark.parametrize("N,V,dtype", [
    (40, 128256, torch.float32),      # 513 KB rows: eight CTAs of 64 KB
    (24, 256000, torch.bfloat16),     # 512 KB rows
    (12, 256000, torch.float32),      # 1 MB rows: eight CTAs of 128 KB, one per SM
    (300, 8, torch.bfloat16),         # one vector per row: seven of a CTA's eight warps have nothing to fetch
    (70, 50264, torch.float16),       # two CTAs of 50 KB; pieces and the last slice are ragged
    (9, 409600, torch.float32),       # 1.6 MB rows: the largest the cluster form takes
])
def test_ce_cluster_form_geometries(N, V, dtype):
    """Row lengths that exercise every cluster size of the one-launch form, its short last slices and idle warps; the
    launch count shows that this form ran (count, cluster kernel, reduction = 3 launches, the fold-in of the upstream gradient 1)."""
    from liger_kernel_b200 import _lib
    from oracle.flce_oracle import ce_oracle

    logits, t = ce_cases.random_case(N, V, dtype, dict())
    kw = dict(label_smoothing=0.05, lse_square_scale=1e-4)
    torch.cuda.synchronize()
    before = _lib.lib.flce_b200_kernel_launches()
    res = ce_cases.run_ce(logits, t, "cuda", mode="auto", grad_output=0.5, **kw)
    assert _lib.lib.flce_b200_kernel_launches() - before == 4
    ce_cases.check_ce(res, ce_oracle(logits, t, grad_output=0.5, **kw), dtype)
    two = ce_cases.run_ce(logits, t, "cuda", mode="two_pass", grad_output=0.5, **kw)
    assert torch.equal(res["predicted"], two["predicted"])
    assert _lib.lib.flce_b200_check_device_status(None) == 0


def test_ce_cluster_form_declines_what_it_cannot_hold():
    """Rows longer than eight CTAs' shared memory, or not a multiple of 16 bytes, go through the two-pass kernels; asking the
    C entry point for them directly is an error before any launch."""
    import ctypes as C

    from liger_kernel_b200 import _lib
    from liger_kernel_b200.ops import cross_entropy as mod
    from oracle.flce_oracle import ce_oracle

    for N, V, dtype in ((6, 420000, torch.float32), (33, 32001, torch.bfloat16)):
        logits, t = ce_cases.random_case(N, V, dtype, dict())
        before = _lib.lib.flce_b200_kernel_launches()
        res = ce_cases.run_ce(logits, t, "cuda", mode="auto")
        assert _lib.lib.flce_b200_kernel_launches() - before == 6
        ce_cases.check_ce(res, ce_oracle(logits, t), dtype)
        prep = mod._CePrepared(logits.cuda(), t.cuda(), None, -100, 0.0, 0.0, "mean", None)
        dummy = torch.empty(64, device="cuda")
        rc = _lib.lib.flce_b200_ce_forward_backward(C.byref(prep.problem), dummy.data_ptr(), dummy.data_ptr(),
                                                    C.byref(_lib.ForwardOut()), prep.logits.data_ptr(), V, None)
        assert rc == _lib.FLCE_ERR_UNSUPPORTED


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
