"""Host-side glue that needs no GPU: rebinding the operator inside an importable liger_kernel package, running the
loss from inside an FSDP-style wrapper's forward, and the reduction / return-type conventions of the loss helpers."""

import sys
import types

import pytest
import torch


def _fake_liger(monkeypatch):
    """A stand-in for an installed liger_kernel with the three modules that bind the operator at import time."""
    names = ["liger_kernel", "liger_kernel.ops", "liger_kernel.transformers", "liger_kernel.transformers.functional",
             "liger_kernel.transformers.fused_linear_cross_entropy"]
    mods = {n: types.ModuleType(n) for n in names}
    for n in names[1:]:
        parent, child = n.rsplit(".", 1)
        setattr(mods[parent], child, mods[n])
    sentinel = object()
    for n in (names[1], names[3], names[4]):
        mods[n].LigerFusedLinearCrossEntropyFunction = sentinel
    for n, m in mods.items():
        monkeypatch.setitem(sys.modules, n, m)
    return mods, sentinel


def test_install_rebinds_the_three_import_sites(monkeypatch):
    import liger_kernel_b200 as lk

    mods, sentinel = _fake_liger(monkeypatch)
    assert lk.install() is True
    for n in ("liger_kernel.ops", "liger_kernel.transformers.functional", "liger_kernel.transformers.fused_linear_cross_entropy"):
        assert mods[n].LigerFusedLinearCrossEntropyFunction is lk.LigerFusedLinearCrossEntropyFunction
        assert mods[n].LigerFusedLinearCrossEntropyFunction is not sentinel


def test_install_on_request_rebinds_the_sibling_operators(monkeypatch):
    import liger_kernel_b200 as lk

    mods, sentinel = _fake_liger(monkeypatch)
    for n in ("liger_kernel.transformers.cross_entropy", "liger_kernel.transformers.fused_linear_jsd"):
        mods[n] = types.ModuleType(n)
        setattr(mods["liger_kernel.transformers"], n.rsplit(".", 1)[1], mods[n])
        monkeypatch.setitem(sys.modules, n, mods[n])
    assert lk.install(cross_entropy=True, fused_linear_jsd=True, fused_linear_scaled_cross_entropy=True) is True
    assert mods["liger_kernel.transformers.cross_entropy"].LigerCrossEntropyFunction is lk.LigerCrossEntropyFunction
    assert mods["liger_kernel.transformers.fused_linear_jsd"].LigerFusedLinearJSDFunction is lk.LigerFusedLinearJSDFunction
    assert mods["liger_kernel.ops"].LigerFusedLinearScaledCrossEntropyFunction is lk.LigerFusedLinearScaledCrossEntropyFunction
    assert mods["liger_kernel.transformers.functional"].LigerFusedLinearJSDFunction is lk.LigerFusedLinearJSDFunction
    # the default install leaves them alone
    mods2, _ = _fake_liger(monkeypatch)
    assert lk.install() is True and not hasattr(mods2["liger_kernel.ops"], "LigerCrossEntropyFunction")


def test_install_on_request_rebinds_the_preference_losses(monkeypatch):
    import liger_kernel_b200 as lk
    from liger_kernel_b200 import chunked_loss as ours

    mods, _ = _fake_liger(monkeypatch)
    names = ["liger_kernel.chunked_loss", "liger_kernel.chunked_loss.functional"] + [
        f"liger_kernel.chunked_loss.{s}_loss" for s in ("dpo", "orpo", "simpo", "cpo", "kto", "grpo", "jsd", "cosine_similarity")]
    for n in names:
        mods[n] = types.ModuleType(n)
        monkeypatch.setitem(sys.modules, n, mods[n])
    assert lk.install(chunked_loss=True) is True
    assert mods["liger_kernel.chunked_loss"].LigerFusedLinearDPOLoss is ours.LigerFusedLinearDPOLoss
    assert mods["liger_kernel.chunked_loss.kto_loss"].LigerFusedLinearKTOFunction is ours.LigerFusedLinearKTOFunction
    assert mods["liger_kernel.chunked_loss.functional"].liger_fused_linear_simpo == ours.LigerFusedLinearSimPOFunction.apply
    assert (mods["liger_kernel.chunked_loss.functional"].liger_fused_linear_cosine
            == ours.LigerFusedLinearCosineSimilarityFunction.apply)
    mods2, _ = _fake_liger(monkeypatch)                       # a liger_kernel without that sub-package: reported, not raised
    for n in names:
        monkeypatch.delitem(sys.modules, n)
    monkeypatch.setattr(sys, "path", [p for p in sys.path if "baseline/_ref" not in p])
    assert lk.install(chunked_loss=True) is False


def test_install_without_liger_returns_false(monkeypatch):
    import liger_kernel_b200 as lk

    for n in list(sys.modules):
        if n == "liger_kernel" or n.startswith("liger_kernel."):
            monkeypatch.delitem(sys.modules, n)
    monkeypatch.setattr(sys, "path", [p for p in sys.path if "baseline/_ref" not in p])
    monkeypatch.setattr(sys, "meta_path", [_Blocker()] + list(sys.meta_path))
    assert lk.install() is False


class _Blocker:
    """Makes `import liger_kernel` fail even if some copy is installed in the environment."""

    @staticmethod
    def find_spec(name, path=None, target=None):
        if name == "liger_kernel" or name.startswith("liger_kernel."):
            raise ImportError("blocked for the test")
        return None


def test_run_inside_fsdp_forward_calls_fn_while_wrapper_forward_runs():
    from liger_kernel_b200.transformers.fsdp import run_inside_fsdp_forward

    events = []

    class Inner(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.weight = torch.nn.Parameter(torch.ones(3))

        def forward(self, x):
            return x * 2

    class Wrapper(torch.nn.Module):          # behaves like FSDP: gathers parameters around the inner forward
        def __init__(self, inner):
            super().__init__()
            self._fsdp_wrapped_module = inner

        def forward(self, *a, **k):
            events.append("gather")
            try:
                return self._fsdp_wrapped_module(*a, **k)
            finally:
                events.append("reshard")

    inner = Inner()
    wrapper = Wrapper(inner)

    def loss_fn(module, scale):
        events.append("loss")
        assert module.forward(torch.tensor(1.0)) == 2.0     # the real forward is back in place while fn runs
        return module.weight.sum() * scale

    out = run_inside_fsdp_forward(wrapper, loss_fn, inner, 3.0)
    assert float(out.detach()) == 9.0 and events == ["gather", "loss", "reshard"]
    assert inner.forward(torch.tensor(2.0)) == 4.0              # and stays restored afterwards
    with pytest.raises(RuntimeError):
        run_inside_fsdp_forward(wrapper, lambda: (_ for _ in ()).throw(RuntimeError("boom")))
    assert inner.forward(torch.tensor(2.0)) == 4.0


def test_causal_lm_loss_reduction_and_return_types(monkeypatch):
    import liger_kernel_b200.transformers.functional as F
    from liger_kernel_b200.transformers.functional import CrossEntropyOutput
    from liger_kernel_b200.transformers.model.loss_utils import LigerForCausalLMLoss

    seen = {}

    def stand_in(input, weight, target, reduction="mean", ignore_index=-100, softcap=None, accum_dtype=None,
                 return_token_accuracy=False, return_predicted_tokens=False, **kw):
        seen.update(reduction=reduction, target=target.clone(), softcap=softcap, extra=kw)
        loss = torch.tensor(10.0)
        if return_token_accuracy or return_predicted_tokens:
            return CrossEntropyOutput(loss=loss, token_accuracy=torch.tensor(0.25))
        return loss

    monkeypatch.setattr(F, "liger_fused_linear_cross_entropy", stand_in)
    h = torch.zeros(2, 3, 4)
    w = torch.zeros(7, 4)
    labels = torch.tensor([[1, 2, 3], [4, 5, 6]])
    out = LigerForCausalLMLoss(h, w, labels, hidden_size=4, not_a_parameter=1)
    assert float(out) == 10.0 and seen["reduction"] == "mean" and seen["extra"] == {}
    assert seen["target"].tolist() == [2, 3, -100, 5, 6, -100]                      # shifted, padded with ignore_index
    out = LigerForCausalLMLoss(h, w, labels, hidden_size=4, num_items_in_batch=4, final_logit_softcapping=30.0)
    assert float(out) == 2.5 and seen["reduction"] == "sum" and seen["softcap"] == 30.0
    out = LigerForCausalLMLoss(h, w, None, hidden_size=4, shift_labels=labels, return_token_accuracy=True)
    assert isinstance(out, CrossEntropyOutput) and float(out.token_accuracy) == 0.25
    assert seen["target"].tolist() == [1, 2, 3, 4, 5, 6]
