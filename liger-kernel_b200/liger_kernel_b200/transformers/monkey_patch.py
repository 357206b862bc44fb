"""Switch Hugging Face llama / qwen2 / gemma2 causal-LM heads to the fused operator.

Signatures follow ``apply_liger_kernel_to_llama`` / ``_qwen2`` / ``_gemma2`` and
``_apply_liger_kernel_to_instance`` of the reference
(``src/liger_kernel/transformers/monkey_patch.py:221-285, 990-1060, 1598-1660, 3588-3650``).
The ``fused_linear_cross_entropy`` switch and the ``cross_entropy`` switch (logits kept, loss through the
stand-alone cross-entropy operator) are implemented by this package; the other flags (rope, rms_norm,
swiglu / geglu) belong to kernels outside this package and are accepted so existing call sites keep
working: when set they are reported once and otherwise ignored.

``install()`` additionally rebinds the operator symbol inside an installed ``liger_kernel`` so that
code which imports Liger directly (e.g. ``Trainer(use_liger_kernel=True)``) reaches this
implementation.
"""

import inspect
import logging

from types import MethodType

from ..ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction
from .model.causal_lm import gemma2_lce_forward, llama_lce_forward, qwen2_lce_forward

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
    if model is not None:
        model.forward = MethodType(forward_fn, model)
    else:
        getattr(modeling_module, class_name).forward = forward_fn


def apply_liger_kernel_to_llama(rope: bool = True, cross_entropy: bool = False, fused_linear_cross_entropy: bool = True,
                                rms_norm: bool = True, swiglu: bool = True, model=None) -> None:
    assert not (cross_entropy and fused_linear_cross_entropy), (
        "cross_entropy and fused_linear_cross_entropy cannot both be True."
    )
    from transformers.models.llama import modeling_llama

    _report_unhandled(rope=rope, rms_norm=rms_norm, swiglu=swiglu)
    if cross_entropy:
        _patch_cross_entropy()
    if fused_linear_cross_entropy:
        _patch_forward(modeling_llama, "LlamaForCausalLM", llama_lce_forward, model)


def apply_liger_kernel_to_qwen2(rope: bool = True, cross_entropy: bool = False, fused_linear_cross_entropy: bool = True,
                                rms_norm: bool = True, swiglu: bool = True, model=None) -> None:
    assert not (cross_entropy and fused_linear_cross_entropy), (
        "cross_entropy and fused_linear_cross_entropy cannot both be True."
    )
    from transformers.models.qwen2 import modeling_qwen2

    _report_unhandled(rope=rope, rms_norm=rms_norm, swiglu=swiglu)
    if cross_entropy:
        _patch_cross_entropy()
    if fused_linear_cross_entropy:
        _patch_forward(modeling_qwen2, "Qwen2ForCausalLM", qwen2_lce_forward, model)


def apply_liger_kernel_to_gemma2(rope: bool = True, cross_entropy: bool = False, fused_linear_cross_entropy: bool = True,
                                 rms_norm: bool = True, geglu: bool = True, model=None) -> None:
    assert not (cross_entropy and fused_linear_cross_entropy), (
        "cross_entropy and fused_linear_cross_entropy cannot both be True."
    )
    from transformers.models.gemma2 import modeling_gemma2

    _report_unhandled(rope=rope, rms_norm=rms_norm, geglu=geglu)
    if cross_entropy:
        _patch_cross_entropy()
    if fused_linear_cross_entropy:
        _patch_forward(modeling_gemma2, "Gemma2ForCausalLM", gemma2_lce_forward, model)


MODEL_TYPE_TO_APPLY_LIGER_FN = {
    "llama": apply_liger_kernel_to_llama,
    "qwen2": apply_liger_kernel_to_qwen2,
    "gemma2": apply_liger_kernel_to_gemma2,
}


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


def install() -> bool:
    """Rebind ``LigerFusedLinearCrossEntropyFunction`` inside an importable ``liger_kernel`` package
    at the three places that bind it at import time (``liger_kernel.ops``,
    ``liger_kernel.transformers.functional``, ``liger_kernel.transformers.fused_linear_cross_entropy``).
    Returns False when no ``liger_kernel`` is installed."""
    try:
        import liger_kernel.ops as lk_ops
        import liger_kernel.transformers.functional as lk_functional
        import liger_kernel.transformers.fused_linear_cross_entropy as lk_module
    except ImportError:
        return False
    for mod in (lk_ops, lk_functional, lk_module):
        setattr(mod, "LigerFusedLinearCrossEntropyFunction", LigerFusedLinearCrossEntropyFunction)
    return True
