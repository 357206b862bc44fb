"""Tiny Hugging Face causal LMs on the GPU, trained a few steps with and without the fused-linear-cross-entropy
switch: the loss curves must agree.  This is the reference's convergence check in miniature
(test/convergence/bf16/test_mini_models.py: same model, same data, Liger on / off, compare losses); its
tokenised dataset is not available offline, so random token ids stand in."""

import copy

import pytest
import torch

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")


def _tiny(kind):
    common = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                  vocab_size=1031, max_position_embeddings=128)
    if kind == "llama":
        from transformers import LlamaConfig, LlamaForCausalLM
        return LlamaForCausalLM(LlamaConfig(**common))
    if kind == "qwen2":
        from transformers import Qwen2Config, Qwen2ForCausalLM
        return Qwen2ForCausalLM(Qwen2Config(**common))
    from transformers import Gemma2Config, Gemma2ForCausalLM
    return Gemma2ForCausalLM(Gemma2Config(head_dim=16, final_logit_softcapping=30.0, **common))


def _train(model, batches, steps):
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    losses = []
    model.train()
    for i in range(steps):
        ids = batches[i % len(batches)]
        labels = ids.clone()
        labels[:, :3] = -100
        out = model(input_ids=ids, labels=labels)
        assert torch.isfinite(out.loss)
        out.loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        losses.append(float(out.loss.detach()))
    return losses


@pytest.mark.parametrize("kind", ["llama", "qwen2", "gemma2"])
@pytest.mark.parametrize("mode", ["recompute", "single_sweep"])
def test_mini_model_loss_curve_matches_unpatched(kind, mode, monkeypatch):
    import liger_kernel_b200 as lk
    import liger_kernel_b200.ops.fused_linear_cross_entropy as op

    monkeypatch.setattr(op, "MODE", mode)
    torch.manual_seed(0)
    base = _tiny(kind).to(device="cuda", dtype=torch.bfloat16)
    patched = copy.deepcopy(base)
    lk._apply_liger_kernel_to_instance(patched, rope=False, rms_norm=False, swiglu=False, geglu=False)
    g = torch.Generator(device="cuda").manual_seed(1)
    batches = [torch.randint(0, 1031, (4, 48), device="cuda", generator=g) for _ in range(4)]
    want = _train(base, batches, 8)
    got = _train(patched, batches, 8)
    assert patched(input_ids=batches[0], labels=batches[0]).logits is None      # training forward builds no logits
    for a, b in zip(got, want):
        assert abs(a - b) <= 2e-2 * abs(b) + 1e-3, (got, want)
    assert got[-1] < got[0]                                                       # it actually learns
