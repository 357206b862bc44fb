"""Wiring of the model patch layer on CPU: after apply_liger_kernel_to_{llama,qwen2,gemma2} a training forward
must reach liger_fused_linear_cross_entropy with flattened hidden states, shifted labels and the right reduction /
softcap, and must not build logits.  The operator itself is replaced by a recording stand-in (torch math), as the
reference does in test/transformers/test_monkey_patch.py when it checks which forward a model ended up with."""

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _tiny(kind):
    common = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                  vocab_size=97, max_position_embeddings=64)
    if kind == "llama":
        from transformers import LlamaConfig, LlamaForCausalLM
        return LlamaForCausalLM(LlamaConfig(**common))
    if kind == "qwen2":
        from transformers import Qwen2Config, Qwen2ForCausalLM
        return Qwen2ForCausalLM(Qwen2Config(**common))
    from transformers import Gemma2Config, Gemma2ForCausalLM
    return Gemma2ForCausalLM(Gemma2Config(head_dim=8, final_logit_softcapping=30.0, **common))


@pytest.mark.parametrize("kind", ["llama", "qwen2", "gemma2"])
@pytest.mark.parametrize("num_items", [None, 11])
def test_instance_patch_routes_loss_through_flce(kind, num_items, monkeypatch):
    import liger_kernel_b200 as lk
    import liger_kernel_b200.transformers.functional as F

    torch.manual_seed(0)
    model = _tiny(kind)
    calls = []

    def stand_in(input, weight, target, bias=None, reduction="mean", ignore_index=-100, softcap=None, **kw):
        calls.append(dict(shape=tuple(input.shape), wshape=tuple(weight.shape), tshape=tuple(target.shape), reduction=reduction,
                          softcap=softcap, ignore_index=ignore_index))
        logits = (input @ weight.t()).float()
        if softcap is not None:
            logits = softcap * torch.tanh(logits / softcap)
        return torch.nn.functional.cross_entropy(logits, target, ignore_index=ignore_index, reduction=reduction)

    monkeypatch.setattr(F, "liger_fused_linear_cross_entropy", stand_in)
    ids = torch.randint(0, 97, (2, 9))
    labels = ids.clone()
    labels[0, :3] = -100
    model.eval()
    extra = {} if num_items is None else dict(num_items_in_batch=num_items)
    with torch.no_grad():
        want = model(input_ids=ids, labels=labels, **extra).loss
    lk._apply_liger_kernel_to_instance(model, rope=False, rms_norm=False, swiglu=False, geglu=False)
    assert model.forward.__func__.__name__ == "lce_forward"
    model.train()
    out = model(input_ids=ids, labels=labels, **extra)
    assert out.logits is None and len(calls) == 1
    c = calls[0]
    assert c["shape"] == (18, 32) and c["wshape"] == (97, 32) and c["tshape"] == (18,)
    assert c["reduction"] == ("mean" if num_items is None else "sum")
    assert c["softcap"] == (30.0 if kind == "gemma2" else None)
    assert torch.allclose(out.loss, want, rtol=1e-4, atol=1e-5)
    model.eval()
    out = model(input_ids=ids, labels=labels, **extra)       # eval: logits are materialised as usual
    assert out.logits is not None and len(calls) == 1


def test_class_patch_and_flag_conflict():
    import liger_kernel_b200 as lk
    from liger_kernel_b200.transformers.model.causal_lm import llama_lce_forward
    from transformers.models.llama import modeling_llama

    original = modeling_llama.LlamaForCausalLM.forward
    try:
        lk.apply_liger_kernel_to_llama()
        assert modeling_llama.LlamaForCausalLM.forward is llama_lce_forward
    finally:
        modeling_llama.LlamaForCausalLM.forward = original
    with pytest.raises(AssertionError, match="cannot both be True"):
        lk.apply_liger_kernel_to_llama(cross_entropy=True, fused_linear_cross_entropy=True)


def test_loss_utils_shift_and_unpack():
    from liger_kernel_b200.transformers.functional import CrossEntropyOutput
    from liger_kernel_b200.transformers.model.loss_utils import unpack_cross_entropy_result

    t = torch.tensor(1.0)
    assert unpack_cross_entropy_result(t) == (t, None, None, None)
    assert unpack_cross_entropy_result((t, 2)) == (t, 2, None, None)
    o = CrossEntropyOutput(loss=t, token_accuracy=torch.tensor(0.5))
    assert unpack_cross_entropy_result(o)[2] == torch.tensor(0.5)
