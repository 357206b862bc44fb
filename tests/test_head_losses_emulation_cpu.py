"""Fused linear JSD and fused linear scaled cross-entropy end to end on CPU tensors: the Python operators and their chunk
loops run unchanged, the row kernels (csrc/head_loss_kernels.cuh) and the fp32 term split run on the host
(tests/emu/), and the tensor-core GEMM entry point is replaced by torch arithmetic on the same memory
(tests/emu_lib.py).  The case bodies are the GPU test's own (tests/head_loss_cases.py), at sizes the emulation handles
in seconds."""

import pytest
import torch

import emu_lib
import head_loss_cases as cases
from golden_util import jsd_golden_names, sce_golden_names

JSD_GRID = [
    # N, Hs, Ht, V, dtype, beta, temperature, label fraction, ignore_index
    (33, 24, 40, 131, torch.float32, 0.5, 1.0, None, -100),
    (33, 24, 40, 131, torch.bfloat16, 0.5, 1.0, None, -100),
    (33, 24, 40, 131, torch.float16, 0.1, 2.0, 0.3, -100),
    (40, 16, 16, 256, torch.bfloat16, 0.0, 1.0, 0.2, -100),
    (40, 16, 16, 256, torch.float32, 0.0, 0.5, 0.2, 2),
    (40, 31, 17, 203, torch.bfloat16, 1.0, 1.0, 0.2, -100),
    (40, 31, 17, 203, torch.float32, 1.0, 1.5, None, -100),
    (21, 8, 8, 1000, torch.float32, 0.9, 4.0, 0.5, -100),
]


@pytest.mark.parametrize("N,Hs,Ht,V,dtype,beta,temperature,labels,ignore_index", JSD_GRID)
def test_jsd_correctness(monkeypatch, N, Hs, Ht, V, dtype, beta, temperature, labels, ignore_index):
    with emu_lib.installed(monkeypatch):
        cases.case_jsd_correctness("cpu", N, Hs, Ht, V, dtype, beta, temperature, labels, ignore_index)


def test_jsd_functional_and_upstream_gradient(monkeypatch):
    with emu_lib.installed(monkeypatch):
        cases.case_jsd_correctness("cpu", 24, 16, 32, 97, torch.bfloat16, 0.5, 1.0, 0.1, grad_output=2.5, functional=True)
        cases.case_jsd_correctness("cpu", 24, 16, 32, 97, torch.float32, 0.3, 1.0, 0.1, grad_output=0.5)


@pytest.mark.parametrize("name", jsd_golden_names())
def test_jsd_against_reference_golden(monkeypatch, name):
    with emu_lib.installed(monkeypatch):
        cases.case_jsd_golden("cpu", name)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_jsd_multichunk(monkeypatch, dtype):
    with emu_lib.installed(monkeypatch) as lib:
        cases.case_jsd_multichunk_equals_single_chunk("cpu", dtype)
        assert lib.calls.count("flce_b200_jsd_rows") == 1 + 3        # one chunk, then 530 rows in chunks of 256


def test_jsd_all_ignored(monkeypatch):
    with emu_lib.installed(monkeypatch):
        cases.case_jsd_all_ignored("cpu")


def test_jsd_weight_without_grad_and_second_backward(monkeypatch):
    with emu_lib.installed(monkeypatch) as lib:
        cases.case_jsd_weight_without_grad_and_second_backward("cpu")
        # no student-weight gradient requested: logits x2 and grad_input only
        assert lib.calls.count("flce_b200_gemm_accumulate") == 3


SCE_GRID = [
    (17, 31, 257, torch.float32, 1.5, "both"),
    (40, 32, 131, torch.bfloat16, 1.0, "both"),
    (40, 32, 131, torch.float16, 0.7, "nll"),
    (40, 32, 131, torch.bfloat16, 2.0, "entropy"),
    (25, 16, 1000, torch.float32, 0.5, "entropy"),
    (25, 16, 1000, torch.bfloat16, 1.0, "both"),
]


@pytest.mark.parametrize("mode", ["fused", "chunked"])
@pytest.mark.parametrize("N,H,V,dtype,temperature,grads", SCE_GRID)
def test_scaled_ce_correctness(monkeypatch, N, H, V, dtype, temperature, grads, mode):
    if mode == "fused" and dtype == torch.float32:
        pytest.skip("fp32 operands always take the chunked form")
    with emu_lib.installed(monkeypatch) as lib:
        cases.case_sce_correctness("cpu", N, H, V, dtype, temperature, grads, mode=mode)
        assert ("flce_b200_sce_forward" in lib.calls) == (mode == "fused")
        assert ("flce_b200_scaled_ce_rows" in lib.calls) == (mode == "chunked")


@pytest.mark.parametrize("mode", ["fused", "chunked"])
@pytest.mark.parametrize("name", sce_golden_names())
def test_scaled_ce_against_reference_golden(monkeypatch, name, mode):
    with emu_lib.installed(monkeypatch):
        cases.case_sce_golden("cpu", name, mode=mode)


def test_scaled_ce_fused_slabs_and_hidden_padding(monkeypatch):
    """Fused form with a vocabulary that spans several gradient slabs (the stand-in library cuts slabs of 256 classes) and a
    hidden size that needs zero-padding to a multiple of 8; targets in the first, a middle and the last slab."""
    with emu_lib.installed(monkeypatch) as lib:
        cases.case_sce_correctness("cpu", 37, 31, 700, torch.bfloat16, 1.3, "both", mode="fused")
        assert lib.calls.count("flce_b200_sce_backward") == 1


def test_scaled_ce_multichunk_single_output_and_errors(monkeypatch):
    import liger_kernel_b200.ops._chunked as ck

    with emu_lib.installed(monkeypatch) as lib:
        monkeypatch.setattr(ck, "SLAB_BUDGET_BYTES", 256 * ck.slab_pitch(67) * 2)          # 256 rows per chunk
        cases.case_sce_correctness("cpu", 530, 16, 67, torch.bfloat16, 1.25, "both", mode="chunked")
        assert lib.calls.count("flce_b200_scaled_ce_rows") == 3 and lib.calls.count("flce_b200_scaled_ce_grad") == 3
        cases.case_sce_nll_only_output_and_no_grad("cpu")
        cases.case_sce_argument_errors("cpu")


@pytest.mark.parametrize("beta", [0.0, 0.5, 1.0])
def test_jsd_peaked_distributions_stay_finite(monkeypatch, beta):
    """Logit gaps of several hundred (probabilities that underflow fp32) in both heads: loss and gradients stay finite and
    agree with the fp64 closed form, whose own 0 * log 0 terms are defined as 0."""
    import head_loss_cases as cases
    from oracle.distill_oracle import fused_linear_jsd_oracle

    g = torch.Generator().manual_seed(21)
    xs, xt = torch.randn(12, 16, generator=g), torch.randn(12, 16, generator=g)
    ws, wt = torch.randn(97, 16, generator=g) * 6, torch.randn(97, 16, generator=g) * 6
    with emu_lib.installed(monkeypatch):
        res = cases.run_jsd("cpu", xs, ws, xt, wt, None, jsd_beta=beta, temperature=0.25)
    ora = fused_linear_jsd_oracle(xs, ws, xt, wt, None, jsd_beta=beta, temperature=0.25)
    assert bool(torch.isfinite(res["loss"])) and bool(torch.isfinite(res["grad_input"]).all())
    if bool(torch.isfinite(ora.loss)):            # forward / reverse KL are legitimately infinite where a support is missed
        cases.assert_close(res["loss"], ora.loss.float(), 1e-3 * max(1.0, float(ora.loss.abs())), 1e-3, "loss")
        # the gradient is a difference of O(1) terms times |w| / T (about 25 here): fp32 cancellation noise of 1e-5 is expected
        # where the two heads disagree completely and the true gradient vanishes; with reverse KL the terms reach several hundred
        gmax = float(ora.grad_input.abs().max())
        cases.assert_close(res["grad_input"], ora.grad_input.float(), 2e-3 * max(1.0, gmax), 1e-2, "grad_input")


@pytest.mark.parametrize("mode", ["fused", "chunked"])
def test_scaled_ce_peaked_distributions(monkeypatch, mode):
    """Logit gaps of several hundred at a low temperature: entropy near zero, nll in the hundreds, everything finite and equal
    to the fp64 closed form."""
    from oracle.distill_oracle import fused_linear_scaled_ce_oracle

    g = torch.Generator().manual_seed(22)
    x = torch.randn(20, 16, generator=g).bfloat16()
    w = (torch.randn(300, 16, generator=g) * 6).bfloat16()
    t = torch.randint(0, 300, (20,), generator=g)
    t[3] = -100
    g_nll, g_ent = torch.randn(20, generator=g), torch.randn(20, generator=g)
    with emu_lib.installed(monkeypatch), cases.sce_mode(mode):
        res = cases.run_sce("cpu", x, w, t, 0.25, g_nll, g_ent)
    low = torch.bfloat16 if mode == "chunked" else None        # the chunked form rounds its logits slab to the operands' dtype
    ora = fused_linear_scaled_ce_oracle(x, w, t, 0.25, -100, g_nll, g_ent, round_logits_to=low, round_dlogits_to=torch.bfloat16)
    for key in ("nll", "entropy", "grad_input", "grad_weight"):
        assert bool(torch.isfinite(res[key]).all()), key
    cases.assert_close(res["nll"], ora.nll.float(), 1e-3 * float(ora.nll.abs().max()), 1e-3 if low is None else 2e-2, "nll")
    cases.assert_close(res["entropy"], ora.entropy.float(), 2e-2, 2e-2, "entropy")
    gmax = float(ora.grad_input.abs().max())
    cases.assert_close(res["grad_input"], ora.grad_input.float(), 2e-2 * gmax, 5e-2, "grad_input")


def test_jsd_evaluation_pass_skips_the_projections(monkeypatch):
    """Without a gradient to produce (torch.no_grad, or only the head trainable) the chunk loop drops the GEMMs it does not need."""
    import liger_kernel_b200 as lk

    xs, ws, xt, wt, _ = cases.jsd_inputs(40, 16, 16, 67, torch.bfloat16, seed=9)
    with emu_lib.installed(monkeypatch) as lib:
        with torch.no_grad():
            loss = lk.LigerFusedLinearJSD()(xs, ws, xt, wt, None)
        assert lib.calls.count("flce_b200_gemm_accumulate") == 2 and bool(torch.isfinite(loss))
        del lib.calls[:]
        w_train = ws.clone().requires_grad_(True)
        lk.LigerFusedLinearJSD()(xs, w_train, xt, wt, None).backward()
        assert lib.calls.count("flce_b200_gemm_accumulate") == 3 and w_train.grad.shape == (67, 16)      # logits x2 + grad_weight
