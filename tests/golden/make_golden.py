"""Generate the golden vectors in this directory from the reference itself: fused linear cross-entropy (no prefix),
stand-alone cross-entropy (``xent_*``), fused linear JSD (``jsd_*``) and fused linear scaled cross-entropy (``sce_*``).

Run once, in a container that has the reference checkout and no GPU:

    REFERENCE_SRC=<reference checkout>/src python tests/golden/make_golden.py [all|flce|ce|jsd|sce]

For every case below the script
  1. builds seeded inputs,
  2. runs the reference's own ``fused_linear_cross_entropy_forward`` (and, for an
     upstream gradient different from one, ``fused_linear_cross_entropy_backward``)
     on CPU tensors with ``TRITON_INTERPRET=1``, so that the reference's Triton
     kernels (``liger_cross_entropy_kernel``, ``element_mul_kernel``) are executed
     unmodified by Triton's interpreter,
  3. runs the torch ``Linear -> CrossEntropyLoss`` ground truth used by the
     reference's tests through autograd (``ce_weight``/token-scaling cases excepted
     where torch has no equivalent term),
and stores inputs and both sets of outputs in ``<case>.npz``.

Two shims are needed because the interpreter is not the compiler; neither touches
the reference's arithmetic:
  * Python floats passed as kernel arguments have no ``.to`` method in the
    interpreter, so soft-cap values are passed as a ``float`` subclass whose
    ``.to`` returns itself (for the class-weight sums, which the reference obtains
    with ``Tensor.item()``, ``item`` is wrapped for the duration of the call so that
    float results come back as that subclass);
  * libdevice ``tanh`` has no interpreter implementation, so the module-level name
    ``tanh`` of ``liger_kernel.ops.cross_entropy`` is bound to
    ``2*sigmoid(2x)-1`` written with ``triton.language`` primitives.
"""

import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
if "REFERENCE_SRC" not in os.environ:
    raise SystemExit("set REFERENCE_SRC to the src/ directory of the reference checkout")
sys.path.insert(0, os.environ["REFERENCE_SRC"])
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402
import triton.language as tl  # noqa: E402

import liger_kernel.ops.cross_entropy as ref_ce  # noqa: E402
from liger_kernel.ops.fused_linear_cross_entropy import fused_linear_cross_entropy_backward  # noqa: E402
from liger_kernel.ops.fused_linear_cross_entropy import fused_linear_cross_entropy_forward  # noqa: E402

from oracle.flce_oracle import torch_linear_ce_reference  # noqa: E402


class _Float(float):
    def to(self, *_a, **_k):
        return self


@triton.jit
def _interp_tanh(x):
    return 2 * tl.sigmoid(2 * x) - 1


ref_ce.tanh = _interp_tanh

_orig_item = torch.Tensor.item


def _item_with_to(self):
    v = _orig_item(self)
    return _Float(v) if isinstance(v, float) else v

# name -> (N, H, V, dtype, kwargs, extras)
CASES = {
    "mean_default": dict(N=96, H=64, V=257, ign=0.1),
    "sum_default": dict(N=96, H=64, V=257, ign=0.1, reduction="sum"),
    "ragged_odd": dict(N=47, H=31, V=123, ign=0.2),
    "label_smoothing": dict(N=64, H=48, V=203, ign=0.1, label_smoothing=0.1),
    "z_loss": dict(N=64, H=48, V=203, ign=0.1, lse_square_scale=1e-2, return_z_loss=True),
    # V is a power of two here on purpose: the reference pads each vocabulary block with -inf *before*
    # soft-capping, tanh(-inf) = -1 turns the padding into -softcap, and for a small softcap those lanes
    # leak exp(-softcap - max) each into the row's sum-exp.  "softcap_padded_quirk" records that deviation
    # from the torch ground truth (3e-3 on the loss at softcap=3); with softcap=30 it is below fp32 epsilon.
    "softcap": dict(N=64, H=48, V=256, ign=0.1, softcap=3.0, wscale=0.5),
    "softcap_padded_quirk": dict(N=64, H=48, V=203, ign=0.1, softcap=3.0, wscale=0.5),
    "bias": dict(N=64, H=48, V=203, ign=0.1, bias=True),
    "ignore_index_42": dict(N=64, H=48, V=203, ign=0.3, ignore_index=42),
    "all_ignored": dict(N=32, H=48, V=203, ign=1.0),
    "ce_weight": dict(N=64, H=48, V=203, ign=0.1, ce_weight=True, label_smoothing=0.1),
    "token_scaling": dict(N=64, H=48, V=203, ign=0.1, use_token_scaling=True),
    "all_features": dict(
        N=64, H=48, V=203, ign=0.15, bias=True, ce_weight=True, label_smoothing=0.1, ignore_index=42,
        lse_square_scale=1e-4, softcap=30.0, return_z_loss=True, wscale=0.5,
    ),
    "qwen_style": dict(N=128, H=64, V=515, ign=0.2, label_smoothing=0.1, lse_square_scale=1e-4, return_z_loss=True),
    "gemma_style_sum": dict(N=128, H=64, V=515, ign=0.05, softcap=30.0, reduction="sum", wscale=1.0),
    "none_reduction": dict(N=64, H=48, V=203, ign=0.1, reduction="none", token_grad=True),
    "grad_output_2p5": dict(N=64, H=48, V=203, ign=0.1, grad_output=2.5),
    "metrics": dict(N=64, H=48, V=203, ign=0.1, return_token_accuracy=True, return_predicted_tokens=True, wscale=2.0),
    "bf16_mean": dict(N=96, H=64, V=257, ign=0.1, dtype="bfloat16"),
}


def build_inputs(name, spec):
    seed = 1000 + sorted(CASES).index(name)
    g = torch.Generator().manual_seed(seed)
    N, H, V = spec["N"], spec["H"], spec["V"]
    dtype = getattr(torch, spec.get("dtype", "float32"))
    x = torch.randn(N, H, generator=g).to(dtype)
    w = (torch.randn(V, H, generator=g) * spec.get("wscale", 0.1)).to(dtype)
    ignore_index = spec.get("ignore_index", -100)
    t = torch.randint(0, V, (N,), generator=g)
    if ignore_index >= 0:
        t[t == ignore_index] = (ignore_index + 1) % V
    drop = torch.rand(N, generator=g) < spec["ign"]
    if spec["ign"] >= 1.0:
        drop[:] = True
    t[drop] = ignore_index
    bias = (torch.randn(V, generator=g) * 0.5).to(dtype) if spec.get("bias") else None
    cw = (torch.rand(V, generator=g) + 0.5) if spec.get("ce_weight") else None
    tg = (torch.rand(N, generator=g) + 0.5) if spec.get("token_grad") else None
    return x, w, t, bias, cw, tg, ignore_index


def run_case(name, spec):
    x, w, t, bias, cw, tg, ignore_index = build_inputs(name, spec)
    softcap = spec.get("softcap")
    kw = dict(
        ce_weight=cw,
        bias=bias,
        ignore_index=ignore_index,
        lse_square_scale=spec.get("lse_square_scale", 0.0),
        label_smoothing=spec.get("label_smoothing", 0.0),
        reduction=spec.get("reduction", "mean"),
        softcap=None if softcap is None else _Float(softcap),
        return_z_loss=spec.get("return_z_loss", False),
        use_token_scaling=spec.get("use_token_scaling", False),
        return_token_accuracy=spec.get("return_token_accuracy", False),
        return_predicted_tokens=spec.get("return_predicted_tokens", False),
    )
    xr = x.clone().requires_grad_(True)
    wr = w.clone().requires_grad_(True)
    br = None if bias is None else bias.clone().requires_grad_(True)
    kw["bias"] = br
    torch.Tensor.item = _item_with_to
    try:
        with torch.no_grad():  # the operator runs inside an autograd.Function forward
            out = fused_linear_cross_entropy_forward(xr, wr, t, token_grad_output=tg, compute_gradients=True,
                                                     weight_requires_grad=True, **kw)
    finally:
        torch.Tensor.item = _orig_item
    loss, z_loss, acc, pred, gx, gw, gb = out
    go = spec.get("grad_output")
    if go is not None:
        gx, gw, gb = fused_linear_cross_entropy_backward(torch.tensor(go), gx, gw, gb)

    rec = dict(
        x=x.float().numpy(), w=w.float().numpy(), target=t.numpy(),
        ref_loss=loss.float().numpy(), ref_grad_input=gx.float().numpy(), ref_grad_weight=gw.float().numpy(),
    )
    if bias is not None:
        rec["bias"] = bias.float().numpy()
        rec["ref_grad_bias"] = gb.float().numpy()
    if cw is not None:
        rec["ce_weight"] = cw.numpy()
    if tg is not None:
        rec["token_grad"] = tg.numpy()
    if z_loss is not None:
        rec["ref_z_loss"] = z_loss.float().numpy()
    if acc is not None:
        rec["ref_token_accuracy"] = acc.float().numpy()
    if pred is not None:
        rec["ref_predicted_tokens"] = pred.numpy()

    # torch ground truth of the reference's tests (no token-scaling equivalent)
    if not spec.get("use_token_scaling"):
        tl_, tz, tgx, tgw, tgb = torch_linear_ce_reference(
            x, w, t, bias=bias, ce_weight=cw, ignore_index=ignore_index,
            lse_square_scale=kw["lse_square_scale"], label_smoothing=kw["label_smoothing"],
            reduction=kw["reduction"], softcap=softcap, dtype=torch.float32,
        )
        if tg is None and go is None:
            rec["torch_loss"] = tl_.numpy()
            rec["torch_z_loss"] = tz.numpy()
            if spec["ign"] < 1.0:
                rec["torch_grad_input"] = tgx.numpy()
                rec["torch_grad_weight"] = tgw.numpy()
                if tgb is not None:
                    rec["torch_grad_bias"] = tgb.numpy()
    meta = {k: v for k, v in spec.items()}
    meta["ignore_index"] = ignore_index
    rec["meta"] = np.array(repr(meta))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
    print(f"{name}: loss={np.asarray(rec['ref_loss']).reshape(-1)[:1]}")


# ---- stand-alone cross-entropy on materialised logits: the reference's cross_entropy_forward / _backward ---------
CE_CASES = {
    "xent_mean_default": dict(N=64, V=203, ign=0.1),
    "xent_sum_bf16": dict(N=64, V=256, ign=0.1, reduction="sum", dtype="bfloat16"),
    "xent_none_token_grad": dict(N=48, V=131, ign=0.2, reduction="none", token_grad=True),
    "xent_all_features": dict(N=64, V=256, ign=0.15, weight=True, label_smoothing=0.1, ignore_index=42, lse_square_scale=1e-3,
                            softcap=30.0, return_z_loss=True, scale=4.0),
    "xent_metrics_grad_output": dict(N=64, V=515, ign=0.1, return_token_accuracy=True, return_predicted_tokens=True,
                                   grad_output=0.5, scale=3.0),
}


def run_ce_case(name, spec):
    from liger_kernel.ops.cross_entropy import cross_entropy_backward, cross_entropy_forward

    seed = 2000 + sorted(CE_CASES).index(name)
    g = torch.Generator().manual_seed(seed)
    N, V = spec["N"], spec["V"]
    dtype = getattr(torch, spec.get("dtype", "float32"))
    logits = (torch.randn(N, V, generator=g) * spec.get("scale", 2.0)).to(dtype)
    ignore_index = spec.get("ignore_index", -100)
    t = torch.randint(0, V, (N,), generator=g)
    if ignore_index >= 0:
        t[t == ignore_index] = (ignore_index + 1) % V
    t[torch.rand(N, generator=g) < spec["ign"]] = ignore_index
    weight = (torch.rand(V, generator=g) + 0.5) if spec.get("weight") else None
    tg = (torch.rand(N, generator=g) + 0.5) if spec.get("token_grad") else None
    softcap = spec.get("softcap")
    work = logits.clone().requires_grad_(True)
    torch.Tensor.item = _item_with_to
    try:
        with torch.no_grad():
            loss, z_loss, acc, pred, grad = cross_entropy_forward(
                work, t, weight, ignore_index, spec.get("lse_square_scale", 0.0), spec.get("label_smoothing", 0.0),
                spec.get("reduction", "mean"), None if softcap is None else _Float(softcap), spec.get("return_z_loss", False),
                spec.get("return_token_accuracy", False), spec.get("return_predicted_tokens", False))
            if tg is not None:
                grad = cross_entropy_backward(grad, tg.to(dtype))
            elif spec.get("grad_output") is not None:
                grad = cross_entropy_backward(grad, torch.tensor(spec["grad_output"], dtype=dtype))
    finally:
        torch.Tensor.item = _orig_item
    rec = dict(logits=logits.float().numpy(), target=t.numpy(), ref_loss=loss.float().numpy(),
               ref_grad_logits=grad.detach().float().numpy())
    if weight is not None:
        rec["weight"] = weight.numpy()
    if tg is not None:
        rec["token_grad"] = tg.numpy()
    if z_loss is not None:
        rec["ref_z_loss"] = z_loss.float().numpy()
    if acc is not None:
        rec["ref_token_accuracy"] = acc.float().numpy()
    if pred is not None:
        rec["ref_predicted_tokens"] = pred.numpy()
    meta = dict(spec)
    meta["ignore_index"] = ignore_index
    rec["meta"] = np.array(repr(meta))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
    print(f"{name}: loss={np.asarray(rec['ref_loss']).reshape(-1)[:1]}")


# ---- fused linear JSD: the reference's fused_linear_jsd_forward / _backward (Triton _jsd_kernel under the interpreter) ---
JSD_CASES = {
    "jsd_default": dict(N=48, Hs=32, Ht=64, V=131),
    "jsd_labels_beta01_t2": dict(N=48, Hs=32, Ht=64, V=131, labels=0.25, beta=0.1, temperature=2.0),
    "jsd_forward_kl": dict(N=40, Hs=24, Ht=24, V=203, labels=0.1, beta=0.0),
    "jsd_reverse_kl": dict(N=40, Hs=24, Ht=24, V=203, labels=0.1, beta=1.0, temperature=0.5),
    "jsd_bf16_grad_output": dict(N=64, Hs=32, Ht=64, V=256, labels=0.1, beta=0.5, dtype="bfloat16", grad_output=2.5),
    "jsd_ignore_index_7": dict(N=40, Hs=24, Ht=48, V=97, labels=0.3, beta=0.7, ignore_index=7, temperature=1.5),
}


def run_jsd_case(name, spec):
    from liger_kernel.ops.fused_linear_jsd import fused_linear_jsd_backward, fused_linear_jsd_forward

    seed = 3000 + sorted(JSD_CASES).index(name)
    g = torch.Generator().manual_seed(seed)
    N, Hs, Ht, V = spec["N"], spec["Hs"], spec["Ht"], spec["V"]
    dtype = getattr(torch, spec.get("dtype", "float32"))
    xs = torch.randn(N, Hs, generator=g).to(dtype)
    ws = (torch.randn(V, Hs, generator=g) * 0.3).to(dtype)
    xt = torch.randn(N, Ht, generator=g).to(dtype)
    wt = (torch.randn(V, Ht, generator=g) * 0.3).to(dtype)
    ignore_index = spec.get("ignore_index", -100)
    labels = None
    if "labels" in spec:
        labels = torch.randint(0, V, (N,), generator=g)
        if ignore_index >= 0:
            labels[labels == ignore_index] = (ignore_index + 1) % V
        labels[torch.rand(N, generator=g) < spec["labels"]] = ignore_index
    xr, wr = xs.clone().requires_grad_(True), ws.clone().requires_grad_(True)
    with torch.no_grad():
        loss, gx, gw = fused_linear_jsd_forward(xr, wr, xt, wt, labels, spec.get("beta", 0.5), ignore_index, labels is not None,
                                                spec.get("temperature", 1.0))
        if spec.get("grad_output") is not None:
            gx, gw = fused_linear_jsd_backward(torch.tensor(spec["grad_output"]), gx, gw)
    rec = dict(student_input=xs.float().numpy(), student_weight=ws.float().numpy(), teacher_input=xt.float().numpy(),
               teacher_weight=wt.float().numpy(), ref_loss=loss.float().numpy(), ref_grad_input=gx.float().numpy(),
               ref_grad_weight=gw.float().numpy())
    if labels is not None:
        rec["labels"] = labels.numpy()
    meta = dict(spec)
    meta["ignore_index"] = ignore_index
    rec["meta"] = np.array(repr(meta))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
    print(f"{name}: loss={np.asarray(rec['ref_loss']).reshape(-1)[:1]}")


# ---- fused linear scaled cross-entropy: the reference's device-independent implementation, run on CPU tensors -------------
SCE_CASES = {
    "sce_fp32_ragged_both": dict(N=37, H=31, V=257, temperature=1.5, ign=0.2, grads="both"),
    "sce_nll_only": dict(N=40, H=32, V=131, temperature=1.0, ign=0.1, grads="nll"),
    "sce_entropy_only": dict(N=40, H=32, V=131, temperature=0.7, ign=0.1, grads="entropy"),
    "sce_bf16_both": dict(N=64, H=64, V=256, temperature=2.0, ign=0.1, grads="both", dtype="bfloat16"),
    "sce_multichunk": dict(N=600, H=16, V=67, temperature=1.25, ign=0.05, grads="both"),      # spans two 512-token chunks
}


def run_sce_case(name, spec):
    from liger_kernel.ops.fused_linear_scaled_cross_entropy import LigerFusedLinearScaledCrossEntropyFunction

    seed = 4000 + sorted(SCE_CASES).index(name)
    g = torch.Generator().manual_seed(seed)
    N, H, V = spec["N"], spec["H"], spec["V"]
    dtype = getattr(torch, spec.get("dtype", "float32"))
    x = (torch.randn(N, H, generator=g) * 0.5).to(dtype)
    w = (torch.randn(V, H, generator=g) / H ** 0.5 * 2).to(dtype)
    t = torch.randint(0, V, (N,), generator=g)
    t[torch.rand(N, generator=g) < spec["ign"]] = -100
    g_nll = torch.randn(N, generator=g)
    g_ent = torch.randn(N, generator=g)
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    nll, entropy = LigerFusedLinearScaledCrossEntropyFunction.apply(xr, wr, t, spec["temperature"], -100, 1, True)
    total = 0
    if spec["grads"] in ("both", "nll"):
        total = total + (nll * g_nll).sum()
    if spec["grads"] in ("both", "entropy"):
        total = total + (entropy.float() * g_ent).sum()
    total.backward()
    rec = dict(x=x.float().numpy(), w=w.float().numpy(), target=t.numpy(), grad_nll=g_nll.numpy(), grad_entropy=g_ent.numpy(),
               ref_nll=nll.detach().float().numpy(), ref_entropy=entropy.detach().float().numpy(),
               ref_grad_input=xr.grad.float().numpy(), ref_grad_weight=wr.grad.float().numpy())
    meta = dict(spec)
    meta["ignore_index"] = -100
    rec["meta"] = np.array(repr(meta))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
    print(f"{name}: nll[:2]={rec['ref_nll'][:2]} entropy[:2]={rec['ref_entropy'][:2]}")


if __name__ == "__main__":
    which = sys.argv[1] if len(sys.argv) > 1 else "all"       # all | flce | ce | jsd | sce
    if which in ("all", "flce"):
        for case_name in sorted(CASES):
            run_case(case_name, CASES[case_name])
    if which in ("all", "ce"):
        for case_name in sorted(CE_CASES):
            run_ce_case(case_name, CE_CASES[case_name])
    if which in ("all", "jsd"):
        for case_name in sorted(JSD_CASES):
            run_jsd_case(case_name, JSD_CASES[case_name])
    if which in ("all", "sce"):
        for case_name in sorted(SCE_CASES):
            run_sce_case(case_name, SCE_CASES[case_name])
