"""bench_ops.py (timing of the operators beside the headline path) driven on CPU tensors through the kernel emulation:
the three operator steps run, the JSON record has the contract's keys, and the work model matches the shapes."""

import json

import pytest
import torch

import emu_lib


@pytest.mark.parametrize("op,rows,hidden,vocab", [("ce", 6, 0, 203), ("jsd", 5, 32, 131), ("scaled_ce", 5, 24, 131)])
def test_bench_ops_record(monkeypatch, op, rows, hidden, vocab):
    import bench_ops

    with emu_lib.installed(monkeypatch):
        rec = bench_ops.run(op, "ours", rows, hidden, vocab, torch.bfloat16, steps=2, warmup=1, device=torch.device("cpu"))
    json.dumps(rec)
    for key in ("op", "impl", "metric", "value", "unit", "ms_per_step", "steps", "warmup", "n_gpus", "higher_is_better", "dtype",
                "data", "config", "roofline", "gpu_launches", "clocks"):
        assert key in rec, key
    assert rec["value"] > 0 and rec["ms_per_step"] > 0 and rec["roofline"]["frac"] > 0
    assert rec["roofline"]["bound"] == ("hbm" if op == "ce" else "tensor")
    bound, units = bench_ops.work_per_step(op, rows, hidden, vocab, 2)
    if op == "ce":
        assert units == 2 * rows * vocab * 2          # each logit read once, each gradient written once
    elif op == "jsd":
        assert units == 2 * rows * vocab * (hidden // 2 + hidden) + 4 * rows * vocab * (hidden // 2)
    else:
        assert units == 8 * rows * hidden * vocab
    assert rec["last_loss"] == rec["last_loss"]          # finite / not NaN


def test_bench_inputs_zipf_targets_for_the_gemma_style_workload():
    """bench.py's config C4 draws targets from a Zipf(1.1) law over the class ranks; the other workloads stay uniform."""
    import bench

    assert bench.WORKLOADS["c4"]["zipf"] == 1.1 and "zipf" not in bench.WORKLOADS["c2"]
    spec = dict(N=40000, H=8, V=1000, ign=0.05, zipf=1.1, kw={})
    x, w, t = bench.make_inputs(spec, torch.device("cpu"), 1)
    assert x.shape == (40000, 8) and x.dtype == torch.bfloat16 and w.shape == (1000, 8)
    live = t[t >= 0]
    counts = torch.bincount(live, minlength=1000).double()
    assert 1.9 < float(counts[0] / counts[1]) < 2.4                       # 2^1.1 = 2.14
    assert 10.0 < float(counts[0] / counts[9]) < 16.0                     # 10^1.1 = 12.6
    assert int(live.max()) <= 999 and 0.04 < float((t == -100).float().mean()) < 0.06
    uniform = bench.make_inputs(dict(N=40000, H=8, V=1000, ign=0.05, kw={}), torch.device("cpu"), 1)[2]
    u = torch.bincount(uniform[uniform >= 0], minlength=1000).double()
    assert float(u.max() / u.min()) < 6.0 and float(counts.max() / max(1.0, float(counts[500:].mean()))) > 100.0


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` (the CPU arm of the headline benchmark) needs no GPU: one JSON line with the contract's keys."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    done = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--workload", "small", "--steps", "1",
                           "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=root)
    assert done.returncode == 0, done.stderr[-2000:]
    rec = json.loads(done.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and rec["metric"] == "flce_fwd_bwd_tokens_per_s" and rec["unit"] == "tokens/s"
    assert rec["value"] > 0 and rec["higher_is_better"] is True and rec["n_gpus"] == 1 and rec["steps"] == 1
    assert rec["cpu_baseline"]["kind"] == "port" and rec["cpu_baseline"]["cores"] >= 1 and rec["cpu_baseline"]["value"] == rec["value"]
    assert rec["e2e"] == {"value": rec["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in rec["config"] and "sample" in rec["config"]
