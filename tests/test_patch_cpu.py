"""Wiring of the model patch layer on CPU: after apply_liger_kernel_to_<family> a training forward must reach
liger_fused_linear_cross_entropy with flattened hidden states, shifted labels and the right reduction / softcap, must
not build logits, and must return the loss the unpatched Hugging Face model returns (router auxiliary loss included for
mixture-of-experts families).  The operator itself is replaced by a recording stand-in (torch math), as the reference
does in test/transformers/test_monkey_patch.py when it checks which forward a model ended up with."""

import inspect

import pytest
import torch

transformers = pytest.importorskip("transformers")

_COMMON = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
               vocab_size=97, max_position_embeddings=64)
_MOE = dict(num_local_experts=4, num_experts_per_tok=2, output_router_logits=True)

# model_type -> (config class, model class, extra config arguments, soft-cap the operator must receive)
FAMILIES = {
    "llama": ("LlamaConfig", "LlamaForCausalLM", dict(), None),
    "mistral": ("MistralConfig", "MistralForCausalLM", dict(sliding_window=None), None),
    "ministral": ("MinistralConfig", "MinistralForCausalLM", dict(sliding_window=16, head_dim=8), None),
    "mixtral": ("MixtralConfig", "MixtralForCausalLM", dict(_MOE), None),
    "gemma": ("GemmaConfig", "GemmaForCausalLM", dict(head_dim=8), None),
    "gemma2": ("Gemma2Config", "Gemma2ForCausalLM", dict(head_dim=8, final_logit_softcapping=30.0), 30.0),
    "gemma3_text": ("Gemma3TextConfig", "Gemma3ForCausalLM", dict(head_dim=8, final_logit_softcapping=30.0, sliding_window=16), 30.0),
    "qwen2": ("Qwen2Config", "Qwen2ForCausalLM", dict(), None),
    "qwen3": ("Qwen3Config", "Qwen3ForCausalLM", dict(head_dim=8), None),
    "qwen3_moe": ("Qwen3MoeConfig", "Qwen3MoeForCausalLM",
                  dict(head_dim=8, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, output_router_logits=True), None),
    "phi3": ("Phi3Config", "Phi3ForCausalLM", dict(pad_token_id=0), None),
    "olmo2": ("Olmo2Config", "Olmo2ForCausalLM", dict(), None),
    "olmo3": ("Olmo3Config", "Olmo3ForCausalLM", dict(), None),
    "glm4": ("Glm4Config", "Glm4ForCausalLM", dict(head_dim=8, pad_token_id=0), None),
    "smollm3": ("SmolLM3Config", "SmolLM3ForCausalLM", dict(pad_token_id=0), None),
    "nemotron": ("NemotronConfig", "NemotronForCausalLM", dict(), None),
    "exaone4": ("Exaone4Config", "Exaone4ForCausalLM", dict(), None),
    "hunyuan_v1_dense": ("HunYuanDenseV1Config", "HunYuanDenseV1ForCausalLM", dict(head_dim=8, pad_token_id=0), None),
    "hunyuan_v1_moe": ("HunYuanMoEV1Config", "HunYuanMoEV1ForCausalLM", dict(head_dim=8, num_experts=4, moe_topk=2, pad_token_id=0), None),
    "gpt_oss": ("GptOssConfig", "GptOssForCausalLM", dict(_MOE, head_dim=8), None),
    "llama4_text": ("Llama4TextConfig", "Llama4ForCausalLM", dict(head_dim=8, intermediate_size_mlp=64, num_local_experts=2, pad_token_id=0),
                    None),
}


def _tiny(kind):
    config_cls, model_cls, extra, _ = FAMILIES[kind]
    if not hasattr(transformers, model_cls):
        pytest.skip(f"{model_cls} is not in this transformers version")
    return getattr(transformers, model_cls)(getattr(transformers, config_cls)(**dict(_COMMON, **extra)))


def _stand_in(calls):
    def stand_in(input, weight, target, bias=None, reduction="mean", ignore_index=-100, softcap=None, **kw):
        calls.append(dict(shape=tuple(input.shape), wshape=tuple(weight.shape), tshape=tuple(target.shape), reduction=reduction,
                          softcap=softcap, ignore_index=ignore_index))
        logits = (input @ weight.t()).float()
        if softcap is not None:
            logits = softcap * torch.tanh(logits / softcap)
        return torch.nn.functional.cross_entropy(logits, target, ignore_index=ignore_index, reduction=reduction)

    return stand_in


@pytest.mark.parametrize("kind,num_items", [(k, None) for k in FAMILIES] + [("llama", 11), ("qwen2", 11), ("gemma2", 11), ("mixtral", 11)])
def test_instance_patch_routes_loss_through_flce(kind, num_items, monkeypatch):
    import liger_kernel_b200 as lk
    import liger_kernel_b200.transformers.functional as F

    torch.manual_seed(0)
    model = _tiny(kind)
    calls = []
    monkeypatch.setattr(F, "liger_fused_linear_cross_entropy", _stand_in(calls))
    ids = torch.randint(1, 97, (2, 9))
    labels = ids.clone()
    labels[0, :3] = -100
    model.eval()
    extra = {} if num_items is None else dict(num_items_in_batch=num_items)
    with torch.no_grad():
        want = model(input_ids=ids, labels=labels, **extra)
    lk._apply_liger_kernel_to_instance(model, rope=False, rms_norm=False, swiglu=False, geglu=False, relu_squared=False,
                                       layer_norm=False)
    assert model.forward.__func__.__name__ == "lce_forward"
    model.train()
    out = model(input_ids=ids, labels=labels, **extra)
    assert out.logits is None and len(calls) == 1
    c = calls[0]
    assert c["shape"] == (18, 32) and c["wshape"] == (97, 32) and c["tshape"] == (18,)
    assert c["reduction"] == ("mean" if num_items is None else "sum")
    assert c["softcap"] == FAMILIES[kind][3]
    assert torch.allclose(out.loss, want.loss, rtol=1e-4, atol=1e-5)
    if getattr(want, "aux_loss", None) is not None:          # mixture of experts: the router loss is part of the total
        assert torch.allclose(out.aux_loss, want.aux_loss, rtol=1e-5) and out.router_logits is not None
    model.eval()
    out = model(input_ids=ids, labels=labels, **extra)       # eval: logits are materialised as usual
    assert out.logits is not None and len(calls) == 1
    assert torch.allclose(out.loss, want.loss, rtol=1e-5, atol=1e-6)
    out = model(input_ids=ids, labels=labels, return_dict=False, **extra)
    assert torch.allclose(out[0], want.loss, rtol=1e-5, atol=1e-6)


def test_apply_functions_keep_the_reference_signatures():
    """Keyword names, order and defaults of every apply function (the reference's monkey_patch.py definitions)."""
    import liger_kernel_b200 as lk

    def sig(fn):
        return [(p.name, p.default) for p in inspect.signature(fn).parameters.values() if p.kind != p.VAR_KEYWORD]

    std = [("rope", True), ("cross_entropy", False), ("fused_linear_cross_entropy", True), ("rms_norm", True), ("swiglu", True),
           ("model", None)]
    for name in ("llama", "mistral", "ministral", "mixtral", "qwen2", "qwen3", "qwen3_moe", "phi3", "olmo2", "olmo3", "smollm3", "exaone4",
                 "hunyuan_v1_dense", "hunyuan_v1_moe"):
        assert sig(getattr(lk, f"apply_liger_kernel_to_{name}")) == std, name
    geglu = [(n if n != "swiglu" else "geglu", d) for n, d in std]
    for name in ("gemma", "gemma2", "gemma3_text"):
        assert sig(getattr(lk, f"apply_liger_kernel_to_{name}")) == geglu, name
    assert sig(lk.apply_liger_kernel_to_glm4) == [("rope", False)] + std[1:]
    assert sig(lk.apply_liger_kernel_to_gpt_oss) == std[:4] + [("swiglu", False), ("model", None)]
    assert sig(lk.apply_liger_kernel_to_llama4) == std + [("layer_norm", True)]
    assert sig(lk.apply_liger_kernel_to_nemotron) == [("relu_squared", True), ("cross_entropy", False),
                                                      ("fused_linear_cross_entropy", True), ("model", None)]
    assert sig(lk.apply_liger_kernel_to_granite) == [("rope", True), ("cross_entropy", True), ("fused_linear_cross_entropy", False)] + std[3:]
    assert lk.MODEL_TYPE_TO_APPLY_LIGER_FN["llama4"] is lk.MODEL_TYPE_TO_APPLY_LIGER_FN["llama4_text"] is lk.apply_liger_kernel_to_llama4
    lk.apply_liger_kernel_to_nemotron(fused_linear_cross_entropy=False, some_future_flag=True)      # **kwargs are swallowed


def test_granite_offers_only_the_cross_entropy_switch(monkeypatch):
    import liger_kernel_b200 as lk

    with pytest.raises(NotImplementedError, match="not available for Granite"):
        lk.apply_liger_kernel_to_granite(cross_entropy=False, fused_linear_cross_entropy=True)
    monkeypatch.setattr(torch.nn.functional, "cross_entropy", torch.nn.functional.cross_entropy)   # restored at teardown
    lk.apply_liger_kernel_to_granite(rope=False, rms_norm=False, swiglu=False)
    assert torch.nn.functional.cross_entropy is lk.liger_cross_entropy


def test_wrapper_instance_patches_its_language_model():
    """A multimodal wrapper that holds the text decoder as language_model (llama4): the decoder's forward is switched."""
    import liger_kernel_b200 as lk

    decoder = _tiny("llama4_text")

    class Wrapper(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.language_model = decoder

    lk.apply_liger_kernel_to_llama4(rope=False, rms_norm=False, swiglu=False, layer_norm=False, model=Wrapper())
    assert decoder.forward.__func__.__name__ == "lce_forward"
    with pytest.raises(TypeError, match="expected an instance of Llama4ForCausalLM"):
        lk.apply_liger_kernel_to_llama4(model=torch.nn.Linear(2, 2))


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


def test_class_level_patch_for_every_family():
    """Without a model instance the switch rebinds the causal-LM class's forward (and nothing else); restored afterwards."""
    import importlib

    import liger_kernel_b200 as lk
    from liger_kernel_b200.transformers import monkey_patch as mp

    for family in mp._FAMILIES:
        if family.forward is None:
            continue
        try:
            module = importlib.import_module(family.module)
        except ImportError:
            continue
        cls = getattr(module, family.class_name)
        original = cls.forward
        try:
            getattr(lk, f"apply_liger_kernel_to_{family.name}")(**{name: False for name, _ in family.other_flags})
            assert cls.forward is family.forward, family.name
        finally:
            cls.forward = original
