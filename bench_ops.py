#!/usr/bin/env python
"""Forward + backward time of the operators beside the fused linear cross-entropy path, one GPU:

    python bench_ops.py --op ce|jsd|scaled_ce [--impl ours|liger] [--rows N --hidden H --vocab V] [--steps K --warmup W]

  ce         stand-alone cross-entropy on materialised logits [N, V]            (HBM-bound: 3 N V b bytes per step)
  jsd        fused linear JSD, student head H/2 and teacher head H               (tensor-bound)
  scaled_ce  fused linear scaled cross-entropy (nll + entropy, both upstream gradients per token)   (tensor-bound)

Shapes default to the reference's benchmark scripts (benchmark/scripts/benchmark_cross_entropy.py,
benchmark_fused_linear_jsd.py: B*T = 4096 ... 8192 rows, H = 4096, V = 128256); inputs are seeded random tensors, bf16.
`--impl liger` times the unmodified reference from baseline/_ref (its Triton cross-entropy and JSD kernels; for the
scaled cross-entropy the device-independent implementation the reference itself selects on this GPU) on the same
inputs.  One JSON line per run.  `bench.py` stays the benchmark of the headline path; this file measures the rows
that were widened into after it.
"""

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "liger-kernel_b200"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

DEFAULTS = {"ce": dict(rows=8192, hidden=0, vocab=128256), "jsd": dict(rows=4096, hidden=4096, vocab=128256),
            "scaled_ce": dict(rows=8192, hidden=4096, vocab=128256),
            # final RMSNorm + lm_head + cross-entropy; --impl ours_unfused = torch's RMSNorm formula + this library's fused head
            "rmsnorm_head": dict(rows=32768, hidden=4096, vocab=128256),
            # DPO with a reference model on 8 chosen + 8 rejected sequences of rows / 16 tokens (chunked_loss/dpo_loss.py)
            "dpo": dict(rows=16384, hidden=4096, vocab=128256)}


def make_case(op, rows, hidden, vocab, dtype, device, seed=1234):
    g = torch.Generator(device=device).manual_seed(seed)

    def rand(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * scale).to(dtype)

    target = torch.randint(0, vocab, (rows,), generator=g, device=device)
    target = torch.where(torch.rand(rows, generator=g, device=device) < 0.05, torch.full_like(target, -100), target)
    if op == "ce":
        return dict(logits=rand(rows, vocab, scale=2.0), target=target)
    if op == "dpo":
        batch = 16
        t = target.view(batch, rows // batch).clone()
        t[:, : rows // batch // 4] = -100                                       # prompts
        return dict(x=rand(batch, rows // batch, hidden), w=rand(vocab, hidden, scale=0.02),
                    ref_x=rand(batch, rows // batch, hidden), ref_w=rand(vocab, hidden, scale=0.02), target=t)
    if op == "rmsnorm_head":
        return dict(h=rand(rows, hidden, scale=3.0), gamma=(torch.rand(hidden, generator=g, device=device) + 0.5).to(dtype),
                    w=rand(vocab, hidden, scale=0.02), target=target)
    if op == "jsd":
        return dict(xs=rand(rows, hidden // 2), ws=rand(vocab, hidden // 2, scale=0.02), xt=rand(rows, hidden),
                    wt=rand(vocab, hidden, scale=0.02), target=target)
    return dict(x=rand(rows, hidden), w=rand(vocab, hidden, scale=0.02), target=target,
                g_nll=torch.randn(rows, generator=g, device=device), g_ent=torch.randn(rows, generator=g, device=device))


def make_step(op, impl, case, n_calls):
    """Returns a callable running one forward + backward; gradients are dropped between steps.  Both cross-entropy
    implementations write the gradient over the logits they are given, so that operator gets a fresh copy per call,
    made before the clock starts."""
    if impl in ("ours", "ours_unfused"):
        import liger_kernel_b200 as lk

        ce, jsd, sce = lk.liger_cross_entropy, lk.LigerFusedLinearJSD(), lk.LigerFusedLinearScaledCrossEntropyFunction.apply
    else:
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        from liger_kernel.ops.fused_linear_scaled_cross_entropy import LigerFusedLinearScaledCrossEntropyFunction
        from liger_kernel.transformers.functional import liger_cross_entropy as ce
        from liger_kernel.transformers.fused_linear_jsd import LigerFusedLinearJSD

        jsd, sce = LigerFusedLinearJSD(), LigerFusedLinearScaledCrossEntropyFunction.apply
    if op == "dpo":
        x, w = case["x"].requires_grad_(True), case["w"].requires_grad_(True)
        if impl == "ours":
            from liger_kernel_b200.chunked_loss import LigerFusedLinearDPOLoss
        else:
            from liger_kernel.chunked_loss import LigerFusedLinearDPOLoss
        loss_mod = LigerFusedLinearDPOLoss(beta=0.1, use_ref_model=True)

        def step():
            x.grad = w.grad = None
            loss = loss_mod(w, x, case["target"], None, case["ref_x"], case["ref_w"], None)[0]
            loss.backward()
            return loss
        return step
    if op == "rmsnorm_head":
        h, gamma, w = case["h"].requires_grad_(True), case["gamma"].requires_grad_(True), case["w"].requires_grad_(True)
        if impl == "ours":
            def head(hh):
                return lk.liger_fused_rmsnorm_linear_cross_entropy(hh, gamma, w, case["target"], eps=1e-6)
        elif impl == "ours_unfused":
            def head(hh):
                hf = hh.float()
                y = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(hh.dtype) * gamma
                return lk.liger_fused_linear_cross_entropy(y, w, case["target"])
        else:
            from liger_kernel.ops.rms_norm import LigerRMSNormFunction
            from liger_kernel.transformers.functional import liger_fused_linear_cross_entropy as liger_flce

            def head(hh):
                y = LigerRMSNormFunction.apply(hh, gamma, 1e-6, 0.0, "llama", False)
                return liger_flce(y, w, case["target"])

        def step():
            h.grad = gamma.grad = w.grad = None
            loss = head(h)
            loss.backward()
            return loss
        return step
    if op == "ce":
        pool = [case["logits"].clone().requires_grad_(True) for _ in range(n_calls)]

        def step():
            logits = pool.pop()
            loss = ce(logits, case["target"])
            loss.backward()
            return loss
    elif op == "jsd":
        xs, ws = case["xs"].requires_grad_(True), case["ws"].requires_grad_(True)

        def step():
            xs.grad = ws.grad = None
            loss = jsd(xs, ws, case["xt"], case["wt"], case["target"])
            loss.backward()
            return loss
    else:
        x, w = case["x"].requires_grad_(True), case["w"].requires_grad_(True)

        def step():
            x.grad = w.grad = None
            nll, entropy = sce(x, w, case["target"], 1.0, -100, 1, True)
            loss = (nll * case["g_nll"]).sum() + (entropy.float() * case["g_ent"]).sum()
            loss.backward()
            return loss
    return step


def work_per_step(op, rows, hidden, vocab, element_size):
    """(bound, algorithmic units per step): HBM bytes for ce, tensor FLOPs for the two fused heads."""
    if op == "ce":
        # every logit read once, every gradient written once: what both implementations need from HBM when a row stays on
        # chip between its two passes (ours: in a cluster's shared memory; the reference: in L2)
        return "hbm", 2.0 * rows * vocab * element_size
    if op == "dpo":
        return "tensor", 8.0 * rows * hidden * vocab                           # policy: logits + two projections, credited like
                                                                               # the head (plus the reference model's logits)
    if op == "rmsnorm_head":
        return "tensor", 8.0 * rows * hidden * vocab                           # the head's credited FLOPs; the norm is HBM work
    if op == "jsd":
        return "tensor", 2.0 * rows * vocab * (hidden // 2 + hidden) + 4.0 * rows * vocab * (hidden // 2)
    return "tensor", 8.0 * rows * hidden * vocab                           # logits twice (recomputed in backward) + two projections


def time_steps(step, steps, warmup, device):
    for _ in range(warmup):
        step()
    if device.type == "cuda":
        torch.cuda.synchronize(device)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            last = step()
        stop.record()
        torch.cuda.synchronize(device)
        return start.elapsed_time(stop) / steps, float(last.detach())
    t0 = time.perf_counter()
    for _ in range(steps):
        last = step()
    return (time.perf_counter() - t0) * 1e3 / steps, float(last.detach())


def run(op, impl, rows, hidden, vocab, dtype, steps, warmup, device):
    from bench import ClockSampler, load_peaks

    case = make_case(op, rows, hidden, vocab, dtype, device)
    step = make_step(op, impl, case, steps + warmup)
    launches_before = 0
    if impl in ("ours", "ours_unfused"):
        from liger_kernel_b200._lib import lib
        launches_before = lib.flce_b200_kernel_launches()
    if device.type == "cuda":
        with ClockSampler(device.index or 0) as sampler:
            ms, loss = time_steps(step, steps, warmup, device)
        clocks = sampler.summary()
    else:
        ms, loss = time_steps(step, steps, warmup, device)
        clocks = None
    launches = None
    if impl in ("ours", "ours_unfused"):
        launches = (lib.flce_b200_kernel_launches() - launches_before) * steps // (steps + warmup)
    bound, units = work_per_step(op, rows, hidden, vocab, torch.empty((), dtype=dtype).element_size())
    peaks = load_peaks()
    achieved = units / (ms * 1e-3) / (1e9 if bound == "hbm" else 1e12)
    peak = peaks["hbm"] if bound == "hbm" else peaks["sustained"]
    return {
        "op": op, "impl": impl, "metric": f"{op}_fwd_bwd_tokens_per_s", "value": rows / (ms * 1e-3), "unit": "tokens/s",
        "ms_per_step": ms, "steps": steps, "warmup": warmup, "n_gpus": 1, "higher_is_better": True,
        "dtype": str(dtype).replace("torch.", ""), "data": "synthetic (seeded random tensors, 5 % ignored targets)",
        "config": {"workload": f"{op}: rows={rows} hidden={hidden} vocab={vocab}", "inputs_larger_than_l2": True},
        "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": "GB/s" if bound == "hbm" else "TFLOP/s",
                     "frac": achieved / peak, "traffic": None, "peak_source": peaks["source"]},
        "gpu_launches": launches, "clocks": clocks, "last_loss": loss,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=sorted(DEFAULTS))
    ap.add_argument("--impl", default="ours", choices=["ours", "ours_unfused", "liger"])
    ap.add_argument("--rows", type=int, default=None)
    ap.add_argument("--hidden", type=int, default=None)
    ap.add_argument("--vocab", type=int, default=None)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="library tuning option (flce_b200_set_option), ours only; may be repeated")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    d = DEFAULTS[args.op]
    if not torch.cuda.is_available():
        raise SystemExit("bench_ops.py needs a CUDA device (sm_100a); there is no CPU path")
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    if args.option and args.impl == "ours":
        sys.path.insert(0, os.path.join(ROOT, "liger-kernel_b200"))
        from liger_kernel_b200 import _lib

        for item in args.option:
            name, value = item.split("=", 1)
            _lib.set_option(name, int(value))
    out = run(args.op, args.impl, args.rows or d["rows"], args.hidden if args.hidden is not None else d["hidden"],
              args.vocab or d["vocab"], getattr(torch, args.dtype), args.steps, args.warmup, device)
    if args.option:
        out["options"] = args.option
    print(json.dumps(out))


if __name__ == "__main__":
    main()
