"""The Python host layer on CPU tensors with the shared library replaced by tests/fake_lib.FakeLib: which entry points
are called, in which order, with which shapes / dtypes / pointers, and what the operator hands back.  Covers the
execution modes (recompute, single sweep), fp32 term splits, row compaction for ignored tokens, the stand-alone
cross-entropy operator and the single-process path of the sharded operators."""

import ctypes as C

import pytest
import torch

import fake_lib


def _inputs(N=12, H=31, V=50, dtype=torch.bfloat16, ignored=(1, 4, 5, 9)):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(N, H, generator=g).to(dtype).requires_grad_(True)
    w = torch.randn(V, H, generator=g).to(dtype).requires_grad_(True)
    t = torch.randint(0, V, (N,), generator=g)
    t[list(ignored)] = -100
    return x, w, t


def test_recompute_mode_calls_and_shapes(monkeypatch):
    import liger_kernel_b200.ops.fused_linear_cross_entropy as fl

    with fake_lib.installed(monkeypatch) as fake:
        monkeypatch.setattr(fl, "MODE", "recompute")
        monkeypatch.setattr(fl, "SKIP_IGNORED", False)
        x, w, t = _inputs()
        b = torch.zeros(50, dtype=torch.bfloat16, requires_grad=True)
        loss, z, acc, pred = fl.LigerFusedLinearCrossEntropyFunction.apply(x, w, t, b, None, -100, 1e-4, 0.1, "mean", 30.0, True,
                                                                         None, False, True, True)
        assert fake.calls == ["flce_b200_workspace_bytes", "flce_b200_forward"]
        prob = fake.structs["flce_b200_forward"][0]
        assert (prob.n_rows, prob.hidden, prob.vocab, prob.vocab_total, prob.ld_x) == (12, 32, 50, 50, 32)   # H padded to 8
        assert prob.dtype == 0 and prob.reduction == 0 and prob.flags == 1 and abs(prob.softcap - 30.0) < 1e-6
        assert prob.bias is not None and prob.ce_weight is None and prob.active_rows is None
        assert loss.shape == () and loss.dtype == torch.float32 and z.dtype == torch.bfloat16
        assert acc.shape == () and pred.shape == (12,) and pred.dtype == torch.int64
        loss.backward()
        assert fake.calls[2:] == ["flce_b200_workspace_bytes", "flce_b200_backward"]
        args = fake.structs["flce_b200_backward"][1]
        assert args.grad_dtype == 0 and args.grad_input and args.grad_weight and args.grad_bias and not args.proj_x
        assert x.grad.shape == (12, 31) and x.grad.dtype == torch.bfloat16 and w.grad.shape == (50, 31)
        assert b.grad.shape == (50,) and b.grad.dtype == torch.bfloat16
        # no-grad forward: loss only, and reduction "none" returns rows
        with torch.no_grad():
            rows = fl.LigerFusedLinearCrossEntropyFunction.apply(x, w, t, None, None, -100, 0.0, 0.0, "none")[0]
        assert rows.shape == (12,)


def test_single_sweep_mode_hands_off_then_recomputes(monkeypatch):
    import liger_kernel_b200.ops.fused_linear_cross_entropy as fl

    with fake_lib.installed(monkeypatch) as fake:
        monkeypatch.setattr(fl, "MODE", "single_sweep")
        monkeypatch.setattr(fl, "SKIP_IGNORED", False)
        x, w, t = _inputs(H=32)
        loss = fl.LigerFusedLinearCrossEntropyFunction.apply(x, w, t)[0]
        assert fake.calls == ["flce_b200_workspace_bytes", "flce_b200_forward_backward"]
        loss.backward(retain_graph=True)
        assert fake.calls[2:] == ["flce_b200_scale_gradient", "flce_b200_scale_gradient"]
        loss.backward()
        assert fake.calls[4:] == ["flce_b200_workspace_bytes", "flce_b200_backward"]
        # reduction "none" and fp32 inputs stay on the two-sweep path
        del fake.calls[:]
        fl.LigerFusedLinearCrossEntropyFunction.apply(x, w, t, None, None, -100, 0.0, 0.0, "none")
        assert "flce_b200_forward_backward" not in fake.calls and "flce_b200_forward" in fake.calls


def test_default_mode_compacts_rows_and_forms_gradients_in_forward(monkeypatch):
    """Defaults: ignored rows are moved out of the way and, for mean / sum with 16-bit operands and a gradient wanted,
    forward already forms the gradients; grad_input comes back in token order; backward only scales."""
    import liger_kernel_b200.ops.fused_linear_cross_entropy as fl

    with fake_lib.installed(monkeypatch) as fake:
        assert fl.MODE == "auto" and fl.SKIP_IGNORED
        x, w, t = _inputs(H=32)
        loss = fl.LigerFusedLinearCrossEntropyFunction.apply(x, w, t)[0]
        assert fake.calls == ["flce_b200_compact_rows", "flce_b200_workspace_bytes", "flce_b200_forward_backward",
                              "flce_b200_scatter_rows"]
        prob = fake.structs["flce_b200_forward_backward"][0]
        assert prob.active_rows is not None
        loss.backward()
        assert fake.calls[4:] == ["flce_b200_scale_gradient", "flce_b200_scale_gradient"]
        assert x.grad.shape == (12, 32) and w.grad.shape == (50, 32)
        # forward-only and reduction "none" use the two-sweep path
        del fake.calls[:]
        with torch.no_grad():
            fl.LigerFusedLinearCrossEntropyFunction.apply(x, w, t)
        assert "flce_b200_forward_backward" not in fake.calls and "flce_b200_forward" in fake.calls
        # an in-place change of a saved operand between forward and backward is caught by autograd
        loss = fl.LigerFusedLinearCrossEntropyFunction.apply(x, w, t, None, None, -100, 0.0, 0.0, "none")[0]
        with torch.no_grad():
            w.mul_(2.0)
        with pytest.raises(RuntimeError, match="modified by an inplace operation"):
            loss.sum().backward()


def test_fp32_inputs_use_term_splits_and_fp32_gradients(monkeypatch):
    import liger_kernel_b200.ops.fused_linear_cross_entropy as fl

    with fake_lib.installed(monkeypatch) as fake:
        x, w, t = _inputs(H=20, dtype=torch.float32)
        loss, z, _, _ = fl.LigerFusedLinearCrossEntropyFunction.apply(x, w, t, None, None, -100, 1e-3, 0.0, "mean", None, True)
        assert fake.calls[:4] == ["flce_b200_split_fp32"] * 4
        prob = fake.structs["flce_b200_forward"][0]
        assert prob.dtype == 0 and prob.hidden == 6 * 24 and prob.ld_x == 6 * 24          # 20 -> 24, six term blocks
        assert z.dtype == torch.float32
        loss.backward()
        args = fake.structs["flce_b200_backward"][1]
        assert args.grad_dtype == 2 and args.split_logit_grad == 1 and args.proj_x_cols == 48 and args.lo_cols_w == 24
        assert x.grad.shape == (12, 20) and x.grad.dtype == torch.float32 and w.grad.shape == (50, 20)


def test_ignored_rows_are_compacted_and_results_return_in_token_order(monkeypatch):
    import liger_kernel_b200.ops.fused_linear_cross_entropy as fl

    with fake_lib.installed(monkeypatch) as fake:
        monkeypatch.setattr(fl, "SKIP_IGNORED", True)
        x, w, t = _inputs(H=32)
        live = [i for i in range(12) if i not in (1, 4, 5, 9)]
        order = live + [1, 4, 5, 9]
        seen = {}

        def forward(p, norm, rowstats, out, ws, ws_bytes, stream):
            prob = p._obj
            seen["targets"] = fake_lib.tensor_from(prob.target, 12, torch.int64).clone()
            seen["active"] = int(fake_lib.tensor_from(prob.active_rows, 1, torch.int32)[0])
            fake_lib.float_array(out._obj.loss_rows, 12)[:] = range(12)          # compact row i reports loss i
            fake_lib.tensor_from(out._obj.predicted_tokens, 12, torch.int64)[:] = torch.arange(100, 112)
            return 0

        def backward(p, args, ws, ws_bytes, budget, stream):
            seen["go"] = fake_lib.tensor_from(args._obj.grad_output, 12).clone()
            gx = fake_lib._array(args._obj.grad_input, C.c_uint16, 12 * 32).reshape(12, 32)
            gx[:] = (torch.arange(12)[:, None] + 1).expand(12, 32).to(torch.bfloat16).view(torch.int16).numpy().view("uint16")
            return 0

        fake.hooks["flce_b200_forward"] = forward
        fake.hooks["flce_b200_backward"] = backward
        rows, _, _, pred = fl.LigerFusedLinearCrossEntropyFunction.apply(x, w, t, None, None, -100, 0.0, 0.0, "none", None, False,
                                                                        None, False, False, True)
        assert fake.calls[0] == "flce_b200_compact_rows" and seen["active"] == 8
        assert seen["targets"].tolist() == t[order].tolist()
        # compact row i is token order[i]
        assert [rows[order[i]].item() for i in range(12)] == list(range(12))
        assert [pred[order[i]].item() for i in range(12)] == list(range(100, 112))
        go = torch.arange(12, dtype=torch.float32) * 10
        rows.backward(go)
        assert seen["go"].tolist() == go[order].tolist()                        # per-token gradients follow the rows
        assert fake.calls[-1] == "flce_b200_scatter_rows"
        assert [x.grad[order[i], 0].item() for i in range(8)] == [float(i + 1) for i in range(8)]
        assert float(x.grad[[1, 4, 5, 9]].abs().max()) == 0.0                   # ignored tokens: exact zeros


def test_stand_alone_cross_entropy_operator(monkeypatch):
    import liger_kernel_b200 as lk
    import liger_kernel_b200.ops.cross_entropy as ce

    with fake_lib.installed(monkeypatch) as fake:
        # two-pass form: forward leaves the logits alone, backward writes the gradient over them
        monkeypatch.setattr(ce, "MODE", "two_pass")
        logits = torch.randn(6, 40, dtype=torch.bfloat16, requires_grad=True)
        holder = logits * 1.0
        t = torch.tensor([1, 2, -100, 3, 4, 5])
        out = lk.LigerCrossEntropyLoss(label_smoothing=0.1, return_z_loss=True)(holder, t)
        assert fake.calls == ["flce_b200_ce_forward"]
        prob = fake.structs["flce_b200_ce_forward"][0]
        assert (prob.n_rows, prob.vocab, prob.ld, prob.dtype) == (6, 40, 40, 0) and prob.logits == holder.data_ptr()
        assert out.loss.dtype == torch.bfloat16 and out.z_loss.dtype == torch.bfloat16 and out.token_accuracy is None
        seen = {}

        def ce_backward(p, lse, norm, go, per_row, grad, ld_grad, scratch, stream):
            seen.update(grad=fake_lib._addr(grad), per_row=per_row, ld=ld_grad)
            return 0

        fake.hooks["flce_b200_ce_backward"] = ce_backward
        out.loss.backward(retain_graph=True)
        assert seen == dict(grad=holder.data_ptr(), per_row=0, ld=40)            # gradient lands in the logits' storage
        assert logits.grad.shape == (6, 40)
        with pytest.raises(RuntimeError, match="overwritten"):
            out.loss.backward()
        monkeypatch.setattr(ce, "INPLACE_GRADIENT", False)
        rows = lk.liger_cross_entropy(logits * 1.0, t, reduction="none")
        rows.backward(torch.ones(6))
        assert seen["per_row"] == 1 and seen["grad"] != holder.data_ptr()

        # default form: the gradient is formed in forward (over the logits), backward only folds the upstream gradient in;
        # nothing is formed when nobody records or the logits need no gradient, or when the rows do not qualify
        monkeypatch.setattr(ce, "MODE", "auto")
        monkeypatch.setattr(ce, "INPLACE_GRADIENT", True)
        del fake.calls[:]
        holder = logits * 1.0
        formed = {}

        def ce_forward_backward(p, norm, rowstats, out_, grad, ld_grad, stream):
            formed.update(grad=fake_lib._addr(grad), ld=ld_grad, logits=p._obj.logits)
            return 0

        def ce_scale(grad, ld_grad, n_rows, vocab, dtype, go, per_row, stream):
            formed.update(scaled=fake_lib._addr(grad), shape=(n_rows, vocab, dtype), per_row=per_row)
            return 0

        fake.hooks["flce_b200_ce_forward_backward"] = ce_forward_backward
        fake.hooks["flce_b200_ce_scale_gradient"] = ce_scale
        loss = lk.liger_cross_entropy(holder, t)
        assert fake.calls == ["flce_b200_ce_forward_backward"]
        assert formed == dict(grad=holder.data_ptr(), ld=40, logits=holder.data_ptr())
        loss.backward(retain_graph=True)
        assert fake.calls == ["flce_b200_ce_forward_backward", "flce_b200_ce_scale_gradient"]
        assert formed["scaled"] == holder.data_ptr() and formed["shape"] == (6, 40, 0) and formed["per_row"] == 0
        with pytest.raises(RuntimeError, match="overwritten"):
            loss.backward()
        del fake.calls[:]
        with torch.no_grad():
            lk.liger_cross_entropy(logits * 1.0, t)
        lk.liger_cross_entropy(logits.detach(), t)
        odd = torch.randn(6, 41, dtype=torch.bfloat16, requires_grad=True)        # 82-byte rows: not a multiple of 16 bytes
        lk.liger_cross_entropy(odd * 1.0, t)
        assert fake.calls == ["flce_b200_ce_forward"] * 3
        monkeypatch.setattr(ce, "INPLACE_GRADIENT", False)
        holder = logits * 1.0
        rows = lk.liger_cross_entropy(holder, t, reduction="none")
        rows.backward(torch.ones(6))
        assert formed["per_row"] == 1 and formed["grad"] != holder.data_ptr() and formed["scaled"] == formed["grad"]


def test_sharded_operators_single_process_path(monkeypatch):
    from liger_kernel_b200 import sharded

    with fake_lib.installed(monkeypatch) as fake:
        x, w, t = _inputs(H=32)
        # mean reduction, 16-bit: rows compacted, normalisers counted (and all-reduced when there are ranks), gradients
        # formed in forward with the given normalisers, grad_input back in token order; backward only scales
        loss = sharded.token_sharded_fused_linear_cross_entropy(x, w, t, label_smoothing=0.1)
        assert [c for c in fake.calls if c != "flce_b200_workspace_bytes"] == [
            "flce_b200_compact_rows", "flce_b200_count", "flce_b200_forward_backward", "flce_b200_scatter_rows"]
        loss.backward()
        assert fake.calls[-1] == "flce_b200_scale_gradient" and w.grad.shape == (50, 32)
        # per-token losses: the two-sweep path
        del fake.calls[:]
        x.grad = w.grad = None
        rows = sharded.token_sharded_fused_linear_cross_entropy(x, w, t, reduction="none")
        assert [c for c in fake.calls if c != "flce_b200_workspace_bytes"] == [
            "flce_b200_count", "flce_b200_forward_stats", "flce_b200_forward_finalize"]
        rows.sum().backward()
        assert fake.calls[-1] == "flce_b200_backward" and w.grad.shape == (50, 32)
        del fake.calls[:]
        w_shard = w.detach()[10:30].clone().requires_grad_(True)
        # a vocabulary shard, mean reduction: gradients formed in forward too, fp32 so that the sum over shards rounds once,
        # with the three exchange hooks set
        loss = sharded.vocab_sharded_fused_linear_cross_entropy(x, w_shard, t, 10, 50)
        prob, args = fake.structs["flce_b200_forward_backward"][-2:]
        assert (prob.vocab, prob.vocab_total, prob.vocab_offset, prob.flags) == (20, 50, 10, 1)
        assert args.grad_dtype == 2 and args.norm_given == 1
        assert args.exchange_shift and args.exchange_rowstats and args.after_grad_input
        loss.backward()
        assert w_shard.grad.shape == (20, 32) and w_shard.grad.dtype == torch.bfloat16
        # per-token losses: statistics merged across shards, then the two-sweep backward with fp32 partial grad_input
        del fake.calls[:]
        w_shard.grad = None
        rows = sharded.vocab_sharded_fused_linear_cross_entropy(x, w_shard, t, 10, 50, reduction="none")
        prob = fake.structs["flce_b200_forward_stats"][-1]
        assert (prob.vocab, prob.vocab_total, prob.vocab_offset, prob.flags) == (20, 50, 10, 1)
        rows.sum().backward()
        assert fake.structs["flce_b200_backward"][-1].grad_dtype == 2 and w_shard.grad.shape == (20, 32)


def test_cross_entropy_switch_routes_hf_loss_through_the_operator(monkeypatch):
    """apply_liger_kernel_to_llama(cross_entropy=True) keeps the logits and sends Hugging Face's loss helper to
    liger_cross_entropy (the reference rebinds nn.functional.cross_entropy the same way, monkey_patch.py:191-194)."""
    transformers = pytest.importorskip("transformers")
    import liger_kernel_b200 as lk
    from transformers import LlamaConfig, LlamaForCausalLM

    monkeypatch.setattr(torch.nn.functional, "cross_entropy", torch.nn.functional.cross_entropy)   # restored at teardown
    with fake_lib.installed(monkeypatch) as fake:
        torch.manual_seed(0)
        model = LlamaForCausalLM(LlamaConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
                                             num_key_value_heads=2, vocab_size=97, max_position_embeddings=64))
        lk.apply_liger_kernel_to_llama(rope=False, cross_entropy=True, fused_linear_cross_entropy=False, rms_norm=False,
                                       swiglu=False, model=model)
        assert torch.nn.functional.cross_entropy is lk.liger_cross_entropy
        ids = torch.randint(0, 97, (2, 9))
        out = model(input_ids=ids, labels=ids)
        assert out.logits is not None and "flce_b200_ce_forward" in fake.calls
        prob = fake.structs["flce_b200_ce_forward"][0]
        assert (prob.n_rows, prob.vocab, prob.dtype, prob.reduction) == (18, 97, 2, 0)      # shifted + flattened fp32 logits
