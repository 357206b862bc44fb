"""``forward`` replacements for Hugging Face causal-LM heads that route the training loss through the
fused operator instead of ``lm_head`` + cross-entropy, so the ``[B, T, V]`` logits are never built.

One implementation serves every text decoder in scope; families differ only in whether a final
logit soft-cap is read from the config and whether a router load-balancing loss is added
(mixture-of-experts models).  Behaviour follows the reference's per-model functions, e.g.
``src/liger_kernel/transformers/model/llama.py:24-202``, ``model/qwen2.py:13-130``,
``model/gemma2.py:19-157``, ``model/gemma3.py:20-150``, ``model/mixtral.py:17-167``,
``model/qwen3_moe.py:19-155``, ``model/gpt_oss.py:19-213`` (skip-logits default, ``logits_to_keep``
slicing, ``shift_labels``, PEFT ``modules_to_save`` unwrapping, FSDP forward redirection, extra
``token_accuracy`` / ``predicted_tokens`` outputs, router auxiliary loss).
"""

from dataclasses import dataclass
from typing import Optional

import torch

from transformers.modeling_outputs import CausalLMOutputWithPast, MoeCausalLMOutputWithPast

from ..fsdp import run_inside_fsdp_forward
from .loss_utils import LigerForCausalLMLoss, unpack_cross_entropy_result


@dataclass
class LigerCausalLMOutputWithPast(CausalLMOutputWithPast):
    token_accuracy: Optional[torch.FloatTensor] = None
    predicted_tokens: Optional[torch.LongTensor] = None


@dataclass
class LigerMoeCausalLMOutputWithPast(MoeCausalLMOutputWithPast):
    token_accuracy: Optional[torch.FloatTensor] = None
    predicted_tokens: Optional[torch.LongTensor] = None


def _head_loss(lm_head, hidden_states, hidden_size, labels, shift_labels, **loss_kwargs):
    return LigerForCausalLMLoss(
        hidden_states=hidden_states, lm_head_weight=lm_head.weight, labels=labels, hidden_size=hidden_size,
        shift_labels=shift_labels, **loss_kwargs,
    )


def _loss_through_lm_head(model, hidden_states, labels, shift_labels, **loss_kwargs):
    lm_head = model.lm_head
    try:  # lm_head listed in LoRA's modules_to_save: read the trainable copy
        from peft.utils.other import ModulesToSaveWrapper

        if isinstance(lm_head, ModulesToSaveWrapper):
            lm_head = lm_head.modules_to_save.default
    except ImportError:
        pass
    from torch.distributed.fsdp import FullyShardedDataParallel

    if isinstance(lm_head, FullyShardedDataParallel):
        # the full weight only exists while FSDP's own forward runs: call the loss from inside it
        return run_inside_fsdp_forward(
            lm_head, _head_loss, lm_head.module, hidden_states, model.config.hidden_size, labels, shift_labels,
            **loss_kwargs,
        )
    return _head_loss(lm_head, hidden_states, model.config.hidden_size, labels, shift_labels, **loss_kwargs)


def _make_lce_forward(softcap_from_config: bool = False, moe_balancing_loss=None):
    """``moe_balancing_loss``: None for dense models, else a callable returning the family's
    ``load_balancing_loss_func`` (looked up lazily so that importing this module imports no model code)."""
    moe = moe_balancing_loss is not None

    def lce_forward(
        self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None, inputs_embeds=None,
        labels=None, use_cache=None, output_attentions=None, output_hidden_states=None, output_router_logits=None,
        return_dict=None, cache_position=None, logits_to_keep=0, skip_logits=None, **kwargs,
    ):
        cfg = self.config
        output_attentions = cfg.output_attentions if output_attentions is None else output_attentions
        output_hidden_states = cfg.output_hidden_states if output_hidden_states is None else output_hidden_states
        return_dict = getattr(cfg, "return_dict", True) if return_dict is None else return_dict
        if getattr(cfg, "pretraining_tp", 1) > 1:
            raise Exception("Liger Kernel does not support pretraining_tp!!")
        router = {}
        if moe:
            if output_router_logits is None:
                output_router_logits = getattr(cfg, "output_router_logits", False)
            router = dict(output_router_logits=output_router_logits)

        outputs = self.model(
            input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
            past_key_values=past_key_values, inputs_embeds=inputs_embeds, use_cache=use_cache,
            output_attentions=output_attentions, output_hidden_states=output_hidden_states, return_dict=return_dict,
            cache_position=cache_position, **router, **kwargs,
        )
        hidden_states = outputs[0]
        keep = slice(-logits_to_keep, None) if isinstance(logits_to_keep, int) else logits_to_keep
        kept = hidden_states[:, keep, :]
        shift_labels = kwargs.pop("shift_labels", None)
        have_labels = labels is not None or shift_labels is not None
        if skip_logits and not have_labels:
            raise ValueError("skip_logits is True, but labels and shift_labels are None")
        if skip_logits is None:
            skip_logits = self.training and have_labels
        softcap = getattr(cfg, "final_logit_softcapping", None) if softcap_from_config else None

        logits = loss = token_accuracy = predicted_tokens = None
        if skip_logits:
            extra = dict(final_logit_softcapping=softcap) if softcap_from_config else {}
            result = _loss_through_lm_head(self, kept, labels, shift_labels, **extra, **kwargs)
            loss, _, token_accuracy, predicted_tokens = unpack_cross_entropy_result(result)
        else:
            logits = self.lm_head(kept)
            if softcap is not None:
                logits = torch.tanh(logits / softcap) * softcap
            if have_labels:
                loss = self.loss_function(
                    logits=logits, labels=labels, shift_labels=shift_labels, vocab_size=cfg.vocab_size, **kwargs
                )
        aux_loss = router_logits = None
        if moe and output_router_logits:
            router_logits = outputs.router_logits if return_dict else outputs[-1]
            aux_loss = moe_balancing_loss()(router_logits, self.num_experts, self.num_experts_per_tok, attention_mask)
            if labels is not None:
                loss = loss + self.router_aux_loss_coef * aux_loss.to(loss.device)
        if not return_dict:
            out = (logits,) + tuple(outputs[1:])
            if moe and output_router_logits:
                out = (aux_loss,) + out
            if token_accuracy is not None:
                out = out + (token_accuracy,)
            if predicted_tokens is not None:
                out = out + (predicted_tokens,)
            return (loss,) + out if loss is not None else out
        if moe:
            return LigerMoeCausalLMOutputWithPast(
                loss=loss, aux_loss=aux_loss, logits=logits, past_key_values=outputs.past_key_values,
                hidden_states=outputs.hidden_states, attentions=outputs.attentions,
                router_logits=getattr(outputs, "router_logits", None), token_accuracy=token_accuracy,
                predicted_tokens=predicted_tokens,
            )
        return LigerCausalLMOutputWithPast(
            loss=loss, logits=logits, past_key_values=outputs.past_key_values, hidden_states=outputs.hidden_states,
            attentions=outputs.attentions, token_accuracy=token_accuracy, predicted_tokens=predicted_tokens,
        )

    return lce_forward


def _mixtral_balancing_loss():
    from transformers.models.mixtral.modeling_mixtral import load_balancing_loss_func

    return load_balancing_loss_func


dense_lce_forward = _make_lce_forward()
softcap_lce_forward = _make_lce_forward(softcap_from_config=True)
moe_lce_forward = _make_lce_forward(moe_balancing_loss=_mixtral_balancing_loss)

# the names the first three families were published under
llama_lce_forward = dense_lce_forward
qwen2_lce_forward = dense_lce_forward
gemma2_lce_forward = softcap_lce_forward
