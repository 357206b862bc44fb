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
        assert units == 3 * rows * vocab * 2
    elif op == "jsd":
        assert units == 2 * rows * vocab * (hidden // 2 + hidden) + 4 * rows * vocab * (hidden // 2)
    else:
        assert units == 8 * rows * hidden * vocab
    assert rec["last_loss"] == rec["last_loss"]          # finite / not NaN
