"""Switch Hugging Face causal-LM heads to the fused operator.

Signatures follow the ``apply_liger_kernel_to_<family>`` functions and ``_apply_liger_kernel_to_instance`` of the
reference (``src/liger_kernel/transformers/monkey_patch.py``: llama ``:221-285``, qwen2 ``:990-1060``, gemma2
``:1598-1660``, the model-type table ``:3534-3585``, instance patching ``:3588-3650``).  Covered: the text decoders whose
head is ``hidden_states -> lm_head -> cross-entropy`` (dense, soft-capped and mixture-of-experts); vision-language
wrappers and hybrid state-space models are not.

The ``fused_linear_cross_entropy`` switch and the ``cross_entropy`` switch (logits kept, loss through the
stand-alone cross-entropy operator) are implemented by this package; the other flags (rope, rms_norm,
swiglu / geglu, layer_norm, relu_squared) belong to kernels outside this package and are accepted so existing
call sites keep working: when set they are reported once and otherwise ignored.

``install()`` additionally rebinds the operator symbol inside an installed ``liger_kernel`` so that
code which imports Liger directly (e.g. ``Trainer(use_liger_kernel=True)``) reaches this
implementation.
"""

import importlib
import inspect
import logging

from dataclasses import dataclass
from types import MethodType
from typing import Callable, Optional, Tuple

from ..ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction
from .model.causal_lm import dense_lce_forward, moe_lce_forward, softcap_lce_forward

logger = logging.getLogger(__name__)
_reported = set()


def _report_unhandled(**flags):
    for name, on in flags.items():
        if on and name not in _reported:
            _reported.add(name)
            logger.info("liger_kernel_b200 only provides the fused linear cross-entropy path; '%s=True' is ignored", name)


def _patch_cross_entropy():
    """What the reference does for ``cross_entropy=True`` (``monkey_patch.py:191-194``): the function that Hugging
    Face's loss helpers reach as ``nn.functional.cross_entropy`` becomes ``liger_cross_entropy``."""
    from transformers.loss.loss_utils import nn

    from .functional import liger_cross_entropy

    nn.functional.cross_entropy = liger_cross_entropy


def _patch_forward(modeling_module, class_name, forward_fn, model):
    if model is None:
        getattr(modeling_module, class_name).forward = forward_fn
        return
    target = model
    cls = getattr(modeling_module, class_name)
    if not isinstance(model, cls):
        # a wrapper around the text decoder (e.g. a multimodal model holding it as language_model)
        inner = getattr(model, "language_model", None)
        if not isinstance(inner, cls):
            raise TypeError(f"expected an instance of {class_name}, got {type(model).__name__}")
        target = inner
    target.forward = MethodType(forward_fn, target)


@dataclass(frozen=True)
class _Family:
    """One ``apply_liger_kernel_to_<name>``: where the causal-LM class lives, which forward it gets, and the
    reference's keyword defaults (flags of kernels outside this package included)."""

    name: str
    module: str
    class_name: str
    forward: Optional[Callable]
    other_flags: Tuple[Tuple[str, bool], ...] = (("rope", True), ("rms_norm", True), ("swiglu", True))
    cross_entropy: bool = False
    fused_linear_cross_entropy: bool = True
    extra_kwargs: bool = False        # the reference's function also swallows **kwargs
    model_types: Tuple[str, ...] = ()


_GEGLU = (("rope", True), ("rms_norm", True), ("geglu", True))

_FAMILIES = (
    _Family("llama", "transformers.models.llama.modeling_llama", "LlamaForCausalLM", dense_lce_forward),
    _Family("mistral", "transformers.models.mistral.modeling_mistral", "MistralForCausalLM", dense_lce_forward),
    _Family("ministral", "transformers.models.ministral.modeling_ministral", "MinistralForCausalLM", dense_lce_forward),
    _Family("mixtral", "transformers.models.mixtral.modeling_mixtral", "MixtralForCausalLM", moe_lce_forward),
    _Family("gemma", "transformers.models.gemma.modeling_gemma", "GemmaForCausalLM", dense_lce_forward, _GEGLU),
    _Family("gemma2", "transformers.models.gemma2.modeling_gemma2", "Gemma2ForCausalLM", softcap_lce_forward, _GEGLU),
    _Family("gemma3_text", "transformers.models.gemma3.modeling_gemma3", "Gemma3ForCausalLM", softcap_lce_forward, _GEGLU),
    _Family("qwen2", "transformers.models.qwen2.modeling_qwen2", "Qwen2ForCausalLM", dense_lce_forward),
    _Family("qwen3", "transformers.models.qwen3.modeling_qwen3", "Qwen3ForCausalLM", dense_lce_forward),
    _Family("qwen3_moe", "transformers.models.qwen3_moe.modeling_qwen3_moe", "Qwen3MoeForCausalLM", moe_lce_forward),
    _Family("phi3", "transformers.models.phi3.modeling_phi3", "Phi3ForCausalLM", dense_lce_forward),
    _Family("olmo2", "transformers.models.olmo2.modeling_olmo2", "Olmo2ForCausalLM", dense_lce_forward),
    _Family("olmo3", "transformers.models.olmo3.modeling_olmo3", "Olmo3ForCausalLM", dense_lce_forward),
    _Family("glm4", "transformers.models.glm4.modeling_glm4", "Glm4ForCausalLM", dense_lce_forward,
            (("rope", False), ("rms_norm", True), ("swiglu", True))),
    _Family("smollm3", "transformers.models.smollm3.modeling_smollm3", "SmolLM3ForCausalLM", dense_lce_forward),
    _Family("nemotron", "transformers.models.nemotron.modeling_nemotron", "NemotronForCausalLM", dense_lce_forward,
            (("relu_squared", True),), extra_kwargs=True),
    _Family("exaone4", "transformers.models.exaone4.modeling_exaone4", "Exaone4ForCausalLM", dense_lce_forward),
    _Family("hunyuan_v1_dense", "transformers.models.hunyuan_v1_dense.modeling_hunyuan_v1_dense", "HunYuanDenseV1ForCausalLM",
            dense_lce_forward),
    _Family("hunyuan_v1_moe", "transformers.models.hunyuan_v1_moe.modeling_hunyuan_v1_moe", "HunYuanMoEV1ForCausalLM",
            dense_lce_forward),
    _Family("gpt_oss", "transformers.models.gpt_oss.modeling_gpt_oss", "GptOssForCausalLM", moe_lce_forward,
            (("rope", True), ("rms_norm", True), ("swiglu", False))),
    _Family("llama4", "transformers.models.llama4.modeling_llama4", "Llama4ForCausalLM", dense_lce_forward,
            (("rope", True), ("rms_norm", True), ("swiglu", True), ("layer_norm", True)), model_types=("llama4_text", "llama4")),
    # the reference offers only the cross-entropy switch for granite (its logits are divided by config.logits_scaling)
    _Family("granite", "transformers.models.granite.modeling_granite", "GraniteForCausalLM", None,
            cross_entropy=True, fused_linear_cross_entropy=False),
)


def _make_apply(family: _Family):
    P = inspect.Parameter
    params = [P(name, P.POSITIONAL_OR_KEYWORD, default=default, annotation=bool) for name, default in family.other_flags]
    # the reference's order: other flags first except that cross_entropy / fused_linear_cross_entropy follow the first one
    head, tail = params[:1], params[1:]
    params = head + [P("cross_entropy", P.POSITIONAL_OR_KEYWORD, default=family.cross_entropy, annotation=bool),
                     P("fused_linear_cross_entropy", P.POSITIONAL_OR_KEYWORD, default=family.fused_linear_cross_entropy,
                       annotation=bool)] + tail
    if family.name == "llama4":   # (..., swiglu, model, layer_norm) in the reference
        params = [q for q in params if q.name != "layer_norm"]
        params += [P("model", P.POSITIONAL_OR_KEYWORD, default=None), P("layer_norm", P.POSITIONAL_OR_KEYWORD, default=True)]
    else:
        params.append(P("model", P.POSITIONAL_OR_KEYWORD, default=None))
    if family.extra_kwargs:
        params.append(P("kwargs", P.VAR_KEYWORD))
    signature = inspect.Signature(params, return_annotation=None)

    def apply(*args, **kwargs) -> None:
        bound = signature.bind(*args, **kwargs)
        bound.apply_defaults()
        a = bound.arguments
        assert not (a["cross_entropy"] and a["fused_linear_cross_entropy"]), (
            "cross_entropy and fused_linear_cross_entropy cannot both be True."
        )
        if a["fused_linear_cross_entropy"] and family.forward is None:
            raise NotImplementedError(f"LigerFusedLinearCrossEntropy is not available for {family.name.capitalize()} models.")
        modeling = importlib.import_module(family.module)
        _report_unhandled(**{name: a[name] for name, _ in family.other_flags})
        if a["cross_entropy"]:
            _patch_cross_entropy()
        if a["fused_linear_cross_entropy"]:
            _patch_forward(modeling, family.class_name, family.forward, a["model"])

    apply.__signature__ = signature
    apply.__name__ = apply.__qualname__ = f"apply_liger_kernel_to_{family.name}"
    apply.__doc__ = (f"Route the training loss of ``{family.class_name}`` through the fused operator (class-wide, or one "
                     f"instance when ``model`` is given); keyword defaults are the reference's.")
    return apply


MODEL_TYPE_TO_APPLY_LIGER_FN = {}
for _family in _FAMILIES:
    _fn = _make_apply(_family)
    globals()[_fn.__name__] = _fn
    for _model_type in (_family.model_types or (_family.name,)):
        MODEL_TYPE_TO_APPLY_LIGER_FN[_model_type] = _fn
__all__ = sorted({fn.__name__ for fn in MODEL_TYPE_TO_APPLY_LIGER_FN.values()}) + [
    "MODEL_TYPE_TO_APPLY_LIGER_FN", "_apply_liger_kernel", "_apply_liger_kernel_to_instance", "install"]


def _apply_liger_kernel(model_type: str, **kwargs) -> None:
    if not model_type:
        logger.info("Model type was not provided. No Liger kernels will be applied.")
        return
    if model_type not in MODEL_TYPE_TO_APPLY_LIGER_FN:
        logger.info(f"There are currently no Liger kernels supported for model type: {model_type}.")
        return
    fn = MODEL_TYPE_TO_APPLY_LIGER_FN[model_type]
    accepted = inspect.signature(fn).parameters
    fn(**{k: v for k, v in kwargs.items() if k in accepted})


def _apply_liger_kernel_to_instance(model, **kwargs) -> None:
    model_type = getattr(model, "config", None) and getattr(model.config, "model_type", None)
    if not model_type:
        logger.info("Model type could not be determined from model config. No Liger kernels will be applied.")
        return
    if model_type not in MODEL_TYPE_TO_APPLY_LIGER_FN:
        logger.info(f"There are currently no Liger kernels supported for model type: {model_type}.")
        return
    fn = MODEL_TYPE_TO_APPLY_LIGER_FN[model_type]
    accepted = inspect.signature(fn).parameters
    fn(model=model, **{k: v for k, v in kwargs.items() if k in accepted})


# operator symbol -> modules of an installed liger_kernel that bind it at import time
_INSTALL_SITES = {
    "LigerFusedLinearCrossEntropyFunction": (
        "liger_kernel.ops", "liger_kernel.transformers.functional", "liger_kernel.transformers.fused_linear_cross_entropy"),
    "LigerCrossEntropyFunction": (
        "liger_kernel.ops", "liger_kernel.transformers.functional", "liger_kernel.transformers.cross_entropy"),
    "LigerFusedLinearJSDFunction": (
        "liger_kernel.ops", "liger_kernel.transformers.functional", "liger_kernel.transformers.fused_linear_jsd"),
    "LigerFusedLinearScaledCrossEntropyFunction": ("liger_kernel.ops",),
}


# where the reference binds its preference losses: the defining module, the package and (Functions only, as
# ``liger_fused_linear_<name> = <Function>.apply``) ``chunked_loss/functional.py:10-17``
_PREFERENCE_LOSSES = {"DPO": "dpo", "ORPO": "orpo", "SimPO": "simpo", "CPO": "cpo", "KTO": "kto", "GRPO": "grpo", "JSD": "jsd",
                      "CosineSimilarity": "cosine_similarity"}


def _install_preference_losses() -> bool:
    from .. import chunked_loss as ours

    try:
        package = importlib.import_module("liger_kernel.chunked_loss")
        functional = importlib.import_module("liger_kernel.chunked_loss.functional")
        defining = {short: importlib.import_module(f"liger_kernel.chunked_loss.{short}_loss") for short in _PREFERENCE_LOSSES.values()}
    except ImportError:
        return False
    for name, short in _PREFERENCE_LOSSES.items():
        fn, loss = getattr(ours, f"LigerFusedLinear{name}Function"), getattr(ours, f"LigerFusedLinear{name}Loss")
        setattr(defining[short], f"LigerFusedLinear{name}Function", fn)
        setattr(defining[short], f"LigerFusedLinear{name}Loss", loss)
        setattr(package, f"LigerFusedLinear{name}Loss", loss)
        setattr(functional, f"LigerFusedLinear{name}Function", fn)
        setattr(functional, f"liger_fused_linear_{short.split('_')[0]}", fn.apply)      # ..._cosine for cosine_similarity
    return True


def install(cross_entropy: bool = False, fused_linear_jsd: bool = False, fused_linear_scaled_cross_entropy: bool = False,
            chunked_loss: bool = False) -> bool:
    """Rebind ``LigerFusedLinearCrossEntropyFunction`` inside an importable ``liger_kernel`` package
    at the three places that bind it at import time (``liger_kernel.ops``,
    ``liger_kernel.transformers.functional``, ``liger_kernel.transformers.fused_linear_cross_entropy``), and on request
    the stand-alone cross-entropy, fused linear JSD and fused linear scaled cross-entropy operators at theirs;
    ``chunked_loss=True`` also rebinds the DPO / ORPO / SimPO / CPO / KTO / GRPO / JSD / cosine-similarity classes of ``liger_kernel.chunked_loss``.
    Returns False when no ``liger_kernel`` is installed."""
    from ..ops.cross_entropy import LigerCrossEntropyFunction
    from ..ops.fused_linear_jsd import LigerFusedLinearJSDFunction
    from ..ops.fused_linear_scaled_cross_entropy import LigerFusedLinearScaledCrossEntropyFunction

    wanted = {"LigerFusedLinearCrossEntropyFunction": LigerFusedLinearCrossEntropyFunction}
    if cross_entropy:
        wanted["LigerCrossEntropyFunction"] = LigerCrossEntropyFunction
    if fused_linear_jsd:
        wanted["LigerFusedLinearJSDFunction"] = LigerFusedLinearJSDFunction
    if fused_linear_scaled_cross_entropy:
        wanted["LigerFusedLinearScaledCrossEntropyFunction"] = LigerFusedLinearScaledCrossEntropyFunction
    try:
        modules = {name: importlib.import_module(name) for symbol in wanted for name in _INSTALL_SITES[symbol]}
    except ImportError:
        return False
    for symbol, fn in wanted.items():
        for name in _INSTALL_SITES[symbol]:
            setattr(modules[name], symbol, fn)
    if chunked_loss and not _install_preference_losses():
        return False
    return True
