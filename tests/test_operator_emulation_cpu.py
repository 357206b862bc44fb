"""The fused linear cross-entropy operator end to end on CPU tensors: the Python host layer runs unchanged (argument
checks, hidden-size padding, fp32 term splits, dtype conventions, autograd wiring, row compaction for ignored tokens,
the sharded operators' single-process path), and behind the C ABI the library's own epilogues and row kernels run on the
host with the tcgen05 main loop replaced by a float dot product (tests/emu_lib.py).  Several bodies are the GPU tests'
own (tests/test_flce_gpu.py), called here with tests/flce_cases.DEVICE switched to "cpu"."""

import numpy as np
import pytest
import torch

import emu_lib
import flce_cases
import test_flce_gpu as gpu_tests
from flce_cases import assert_close, make_inputs, oracle_for, run_cuda
from golden_util import golden_names


@pytest.fixture
def emulated(monkeypatch):
    monkeypatch.setattr(flce_cases, "DEVICE", "cpu")
    with emu_lib.installed(monkeypatch) as lib:
        yield lib


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("reduction", ["mean", "sum"])
@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("feat", range(len(gpu_tests.FEATURES)))
def test_correctness_16bit(emulated, dtype, reduction, bias, feat):
    gpu_tests.test_correctness(4, 47, 31, 123, dtype, reduction, bias, gpu_tests.FEATURES[feat])


@pytest.mark.parametrize("reduction", ["mean", "sum"])
@pytest.mark.parametrize("feat", range(len(gpu_tests.FEATURES)))
def test_correctness_fp32_term_splits(emulated, reduction, feat):
    gpu_tests.test_correctness_fp32(4, 47, 31, 123, reduction, True, gpu_tests.FEATURES[feat])
    assert emulated.calls.count("flce_b200_split_fp32") >= 4


@pytest.mark.parametrize("name", golden_names())
def test_against_reference_golden(emulated, name):
    gpu_tests.test_against_reference_golden(name)


@pytest.mark.parametrize("name", ["mean_default", "all_features", "none_reduction", "ce_weight", "ragged_odd", "softcap", "z_loss"])
def test_golden_fp32_inputs_against_reference_outputs(emulated, name):
    """fp32 inputs exactly as the reference saw them, through the term-split path: agreement with the reference's own
    outputs to fp32 accuracy."""
    gpu_tests.test_golden_fp32_inputs_against_reference_outputs(name)


def test_upstream_gradients_weights_scaling_and_edges(emulated):
    gpu_tests.test_grad_output_scalar(2.0)
    gpu_tests.test_reduction_none_per_token_grad()
    gpu_tests.test_token_scaling_and_class_weights()
    gpu_tests.test_all_rows_ignored_exact_zero()
    gpu_tests.test_ignored_rows_have_exact_zero_gradient()
    gpu_tests.test_targets_at_vocab_edges()


def test_multi_slab_backward_equals_single_slab(emulated, monkeypatch):
    import liger_kernel_b200.ops.fused_linear_cross_entropy as mod

    x, w, t, b, _ = make_inputs(150, 32, 1100, torch.bfloat16, seed=2, bias=True)
    one = run_cuda(x, w, t, bias=b, label_smoothing=0.1)
    monkeypatch.setattr(mod, "SLAB_BUDGET_BYTES", 150 * 2 * 256)              # 256 classes per slab -> 5 slabs
    many = run_cuda(x, w, t, bias=b, label_smoothing=0.1)
    assert torch.equal(one["grad_weight"], many["grad_weight"]) and torch.equal(one["grad_bias"], many["grad_bias"])
    gmax = float(one["grad_input"].float().abs().max())
    assert_close(many["grad_input"].float(), one["grad_input"].float(), 8e-3 * gmax, 1e-2, "grad_input across slabs")


@pytest.mark.parametrize("ignored", [0.0, 0.3, 0.97, 1.0])
@pytest.mark.parametrize("reduction", ["mean", "none"])
def test_skipping_ignored_tokens_changes_nothing(emulated, monkeypatch, ignored, reduction):
    """LIGER_B200_FLCE_SKIP_IGNORED: rows are compacted on the device, the sweeps stop at the tiles / k-blocks that still hold
    live rows (scratch beyond them is poisoned with NaN here), and every result comes back in token order."""
    import liger_kernel_b200.ops.fused_linear_cross_entropy as mod

    x, w, t, _, _ = make_inputs(600, 32, 300, torch.bfloat16, seed=7, ignore_frac=ignored)
    if ignored == 1.0:
        t[:] = -100
    go = (torch.rand(600) + 0.5) if reduction == "none" else None
    kw = dict(reduction=reduction, label_smoothing=0.1, lse_square_scale=1e-3)
    plain = run_cuda(x, w, t, grad_output=go, **kw)
    monkeypatch.setattr(mod, "SKIP_IGNORED", True)
    skipped = run_cuda(x, w, t, grad_output=go, **kw)
    assert "flce_b200_compact_rows" in emulated.calls
    for key in ("loss", "z_loss", "token_accuracy", "predicted_tokens", "grad_input"):
        a, b = plain[key].float(), skipped[key].float()
        assert torch.equal(torch.nan_to_num(a), torch.nan_to_num(b)), key
    gmax = max(float(plain["grad_weight"].float().abs().max()), 1e-30)
    assert_close(skipped["grad_weight"].float(), plain["grad_weight"].float(), 8e-3 * gmax, 1e-2, "grad_weight")   # row order of the sum
    assert bool(torch.isfinite(skipped["grad_weight"].float()).all()) and bool(torch.isfinite(skipped["grad_input"].float()).all())
    gpu_tests._check(skipped, oracle_for(x, w, t, grad_output=go, **kw), torch.bfloat16, reduction, 600)


def test_sharded_operators_single_process_numerics(emulated):
    """The token- and vocabulary-sharded operators without a process group: count / statistics / finalize / backward through
    the C ABI one by one (the path every rank runs), equal to the plain operator."""
    from liger_kernel_b200 import sharded

    x, w, t, _, _ = make_inputs(130, 32, 300, torch.bfloat16, seed=11)
    ora = oracle_for(x, w, t, label_smoothing=0.1)
    for fn, extra in ((sharded.token_sharded_fused_linear_cross_entropy, ()), (sharded.vocab_sharded_fused_linear_cross_entropy, (0, 300))):
        xd, wd = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        loss = fn(xd, wd, t, *extra, label_smoothing=0.1)
        loss.backward()
        np.testing.assert_allclose(float(loss.detach()), float(ora.loss), rtol=1e-5)
        for got, want in ((xd.grad, ora.grad_input), (wd.grad, ora.grad_weight)):
            assert_close(got.float(), want.float(), 8e-3 * float(want.abs().max()), 5e-2, "gradient")


def test_logit_gaps_of_several_hundred_stay_finite(emulated):
    """Peaked rows (logits in the hundreds): the online softmax never forms exp of a positive number, the loss is the exact
    gap for confidently wrong rows and 0 for confidently right ones."""
    g = torch.Generator().manual_seed(4)
    x = torch.randn(70, 32, generator=g).bfloat16()
    w = (torch.randn(300, 32, generator=g) * 8).bfloat16()
    t = torch.randint(0, 300, (70,), generator=g)
    logits = x.double() @ w.double().T
    t[:35] = logits[:35].argmax(1)                                   # half of the rows predict their target with certainty
    for kw in (dict(), dict(label_smoothing=0.1, lse_square_scale=1e-4)):
        res = run_cuda(x, w, t, **kw)
        ora = oracle_for(x, w, t, **kw)
        assert bool(torch.isfinite(res["loss"])) and bool(torch.isfinite(res["grad_input"].float()).all())
        assert bool(torch.isfinite(res["grad_weight"].float()).all())
        gpu_tests._check(res, ora, torch.bfloat16, "mean", 70)


def test_exp_store_form_where_it_applies_and_the_redo_path(emulated, monkeypatch):
    """Default single-sweep calls keep exponentials (bf16, no bias gradient, no smoothing under a soft-cap) and logits
    otherwise; ordinary inputs never take the second pass over a chunk, peaked ones do; both forms agree with the oracle."""
    import liger_kernel_b200.ops.fused_linear_cross_entropy as mod

    x, w, t, b, cw = make_inputs(300, 40, 600, torch.bfloat16, seed=11, bias=True, ce_weight=True)
    cases = [(dict(), None, None, "exp"), (dict(label_smoothing=0.1, lse_square_scale=1e-4), None, cw, "exp"),
             (dict(softcap=20.0), None, None, "exp"), (dict(softcap=20.0, label_smoothing=0.1), None, None, "logits"),
             (dict(), b, None, "logits"), (dict(use_token_scaling=True, label_smoothing=0.05), None, None, "exp")]
    for kw, bias, weights, form in cases:
        emulated.store_modes, emulated.redo_chunks = [], 0
        res = run_cuda(x, w, t, bias=bias, ce_weight=weights, **kw)
        assert emulated.store_modes == [form] and emulated.redo_chunks == 0, (kw, emulated.store_modes, emulated.redo_chunks)
        gpu_tests._check(res, oracle_for(x, w, t, bias=bias, ce_weight=weights, **kw), torch.bfloat16, "mean", 300)
    emulated.store_modes = []
    run_cuda(x.half(), w.half(), t)
    assert emulated.store_modes == ["logits"]                       # fp16 cannot hold the exponentials' range
    monkeypatch.setattr(mod, "STORE_MODE", "logits")
    emulated.store_modes = []
    res = run_cuda(x, w, t)
    assert emulated.store_modes == ["logits"]
    gpu_tests._check(res, oracle_for(x, w, t), torch.bfloat16, "mean", 300)
    monkeypatch.setattr(mod, "STORE_MODE", "auto")
    emulated.redo_chunks = 0
    test_logit_gaps_of_several_hundred_stay_finite(emulated)
    assert emulated.redo_chunks >= 1


@pytest.mark.parametrize("ignore_frac", [0.0, 0.5, 0.97])
def test_skip_ignored_gpu_bodies(emulated, monkeypatch, ignore_frac):
    """The bodies of tests/test_flce_skip_ignored_gpu.py at a size the emulation handles."""
    import liger_kernel_b200.ops.fused_linear_cross_entropy as mod
    import test_flce_skip_ignored_gpu as skip_tests

    monkeypatch.setattr(mod, "SKIP_IGNORED", True)
    skip_tests.test_skip_ignored_matches_oracle_and_plain_path(mod, monkeypatch, 300, 31, 123, ignore_frac)
    if ignore_frac == 0.5:
        monkeypatch.setattr(mod, "SKIP_IGNORED", True)
        skip_tests.test_skip_ignored_all_rows_ignored_and_per_token_gradient(mod)


def test_extras_gpu_bodies(emulated, monkeypatch):
    """The bodies of tests/test_flce_full_size_gpu.py: out-of-range targets, the full-size property checks at a reduced size, and
    automatic mixed precision (the CUDA autocast state is simulated: this box has no GPU for torch.autocast to act on)."""
    import test_flce_full_size_gpu as extras

    extras.test_out_of_range_targets_are_counted_and_optionally_raised(monkeypatch)
    monkeypatch.setattr(extras, "FULL_SIZE", {"small_qwen_style": (300, 32, 1300, 0.2, dict(label_smoothing=0.1, lse_square_scale=1e-4)),
                                              "small_gemma_style": (200, 24, 900, 0.05, dict(softcap=30.0, reduction="sum"))})
    for name in extras.FULL_SIZE:
        extras.test_full_size_configs_sampled_against_fp64(name)
    try:
        for amp_dtype in (torch.bfloat16, torch.float16):
            monkeypatch.setattr(torch, "is_autocast_enabled", lambda device_type=None: True)
            monkeypatch.setattr(torch, "get_autocast_dtype", lambda device_type=None, d=amp_dtype: d)
            extras.test_amp_autocast_with_fp32_parameters(amp_dtype)
    finally:
        # torch.autocast saved the simulated "enabled" answer on entry and wrote it back on exit: clear the real state
        torch.set_autocast_enabled("cuda", False)


def test_module_forward_only_structured_output_and_metrics(emulated):
    """After the reference's test_correctness_with_forward_only, test_liger_fused_linear_cross_entropy_structured_output,
    test_correctness_with_token_accuracy and test_correctness_with_predicted_tokens."""
    import liger_kernel_b200 as lk

    x, w, t, b, _ = make_inputs(90, 32, 300, torch.bfloat16, seed=13, bias=True)
    ora = oracle_for(x, w, t, bias=b, lse_square_scale=1e-3)
    with torch.no_grad():
        loss = lk.LigerFusedLinearCrossEntropyLoss()(w, x, t, b)
    assert torch.is_tensor(loss) and not loss.requires_grad and emulated.calls.count("flce_b200_backward") == 0
    assert_close(loss, oracle_for(x, w, t, bias=b).loss.float(), 1e-4, 1e-4, "forward-only loss")
    out = lk.LigerFusedLinearCrossEntropyLoss(lse_square_scale=1e-3, return_z_loss=True, return_token_accuracy=True,
                                              return_predicted_tokens=True)(w, x, t, b)
    assert isinstance(out, lk.CrossEntropyOutput)
    assert_close(out.loss, ora.loss.float(), 1e-4, 1e-4, "loss")
    assert out.z_loss.dtype == torch.bfloat16                                    # z-loss comes back in the operands' dtype
    assert_close(out.z_loss.float(), ora.z_loss.float(), 1e-2 * float(ora.z_loss), 1e-2, "z_loss")
    assert torch.equal(out.predicted_tokens, ora.predicted_tokens)
    np.testing.assert_allclose(float(out.token_accuracy), float(ora.token_accuracy), rtol=1e-6)
    only_loss = lk.liger_fused_linear_cross_entropy(x, w, t, b)
    assert torch.is_tensor(only_loss)


def test_tiny_llama_trains_the_same_with_the_patched_head(emulated):
    """Convergence in miniature (the reference's test/convergence idea): a 2-layer llama takes five optimiser steps with the
    Hugging Face loss and five with the patched forward (fused operator through the emulation); the loss curves coincide."""
    transformers = pytest.importorskip("transformers")
    import copy

    import liger_kernel_b200 as lk

    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, vocab_size=97, max_position_embeddings=64)
    plain = transformers.LlamaForCausalLM(cfg)
    patched = copy.deepcopy(plain)
    lk.apply_liger_kernel_to_llama(rope=False, rms_norm=False, swiglu=False, model=patched)
    g = torch.Generator().manual_seed(1)
    batches = [torch.randint(1, 97, (2, 12), generator=g) for _ in range(5)]
    curves = []
    for model in (plain, patched):
        model.train()
        opt = torch.optim.SGD(model.parameters(), lr=0.05)
        losses = []
        for ids in batches:
            labels = ids.clone()
            labels[:, :3] = -100
            out = model(input_ids=ids, labels=labels)
            opt.zero_grad()
            out.loss.backward()
            opt.step()
            losses.append(float(out.loss.detach()))
        curves.append(losses)
    assert emulated.calls.count("flce_b200_forward") == 5 and emulated.calls.count("flce_b200_backward") == 5
    np.testing.assert_allclose(curves[1], curves[0], rtol=2e-4, atol=2e-4)
    assert curves[0][-1] < curves[0][0]                                          # and it does learn
