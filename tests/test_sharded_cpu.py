"""Cross-rank exchange logic of the sharded FLCE operators on two gloo ranks (CPU), with the CPU stand-in
backend for the local pieces.  Results must equal the oracle's single-process answer for the whole problem.
Mirrors the reference's vocabulary-parallel test (test/megatron/test_cross_entropy.py:593-727: spawn one
process per rank, compare each rank's result with the single-rank cross-entropy)."""

import os
import sys
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def _worker(rank, world, init_file, mode, kw, result_file):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    sys.path.insert(0, os.path.join(os.path.dirname(HERE), "liger-kernel_b200"))
    from cpu_backend import CpuBackend
    from liger_kernel_b200 import sharded
    from oracle.flce_oracle import flce_oracle

    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        N, H, V = 96, 40, 203
        x = torch.randn(N, H, generator=g)
        w = torch.randn(V, H, generator=g) * 0.3
        t = torch.randint(0, V, (N,), generator=g)
        t[::6] = -100
        ora = flce_oracle(x, w, t, **kw)
        if mode == "token":
            lo, hi = rank * N // world, (rank + 1) * N // world
            xs = x[lo:hi].clone().requires_grad_(True)
            ws = w.clone().requires_grad_(True)
            loss = sharded.token_sharded_fused_linear_cross_entropy(xs, ws, t[lo:hi], backend=CpuBackend(), **kw)
            if kw.get("reduction") == "none":
                loss.sum().backward()
                want_loss = ora.loss[lo:hi]
                ora = flce_oracle(x, w, t, grad_output=torch.ones(N), **kw)
            else:
                loss.backward()
                want_loss = ora.loss
            ok = torch.allclose(loss.double(), want_loss, rtol=1e-5, atol=1e-6)
            ok &= torch.allclose(xs.grad.double(), ora.grad_input[lo:hi], rtol=1e-4, atol=1e-7)
            ok &= torch.allclose(ws.grad.double(), ora.grad_weight, rtol=1e-4, atol=1e-7)
        else:
            bounds = [0, 77, V] if world == 2 else [0, V]
            lo, hi = bounds[rank], bounds[rank + 1]
            xs = x.clone().requires_grad_(True)
            ws = w[lo:hi].clone().requires_grad_(True)
            loss = sharded.vocab_sharded_fused_linear_cross_entropy(xs, ws, t, lo, V, backend=CpuBackend(), **kw)
            loss.backward()
            ok = torch.allclose(loss.double(), ora.loss, rtol=1e-5, atol=1e-6)
            ok &= torch.allclose(xs.grad.double(), ora.grad_input, rtol=1e-4, atol=1e-7)
            ok &= torch.allclose(ws.grad.double(), ora.grad_weight[lo:hi], rtol=1e-4, atol=1e-7)
        with open(f"{result_file}.{rank}", "w") as f:
            f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


CASES = [
    ("token", dict()),
    ("token", dict(reduction="sum", label_smoothing=0.1, lse_square_scale=1e-2)),
    ("token", dict(reduction="none")),
    ("vocab", dict()),
    ("vocab", dict(label_smoothing=0.1, lse_square_scale=1e-2, softcap=5.0)),
    ("vocab", dict(reduction="sum")),
]


@pytest.mark.parametrize("mode,kw", CASES)
def test_two_ranks_equal_single_process(mode, kw):
    world = 2
    with tempfile.TemporaryDirectory() as tmp:
        init_file = os.path.join(tmp, "rendezvous")
        result = os.path.join(tmp, "result")
        mp.spawn(_worker, args=(world, init_file, mode, kw, result), nprocs=world, join=True)
        for r in range(world):
            with open(f"{result}.{r}") as f:
                assert f.read() == "ok", f"rank {r}"


def test_merge_rowstats_tie_prefers_lowest_class():
    from liger_kernel_b200.sharded import merge_rowstats

    a = torch.zeros(2, 6, 3)
    a[:, 0] = torch.tensor([[1.0, 5.0, 2.0], [3.0, 5.0, 0.0]])
    a[:, 1] = 1.0
    a[:, 4] = a[:, 0]
    a[0, 5] = torch.tensor([7, 8, 9], dtype=torch.int32).view(torch.float32)
    a[1, 5] = torch.tensor([107, 108, 109], dtype=torch.int32).view(torch.float32)
    m = merge_rowstats(a)
    assert m[0].tolist() == [3.0, 5.0, 2.0]
    assert m[5].view(torch.int32).tolist() == [107, 8, 9]
    assert torch.allclose(m[1], torch.tensor([1 + torch.exp(torch.tensor(-2.0)), 2.0, 1 + torch.exp(torch.tensor(-2.0))]))


# ---- the library's own host path under gloo: gradients formed in forward on every rank, exchanges from inside the sweep
def _emulated_worker(rank, world, init_file, mode, kw, result_file):
    import contextlib

    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    sys.path.insert(0, os.path.join(os.path.dirname(HERE), "liger-kernel_b200"))
    import emu_lib
    import liger_kernel_b200.ops.cross_entropy as ce
    import liger_kernel_b200.ops.fused_linear_cross_entropy as fl
    import liger_kernel_b200.sharded as sh
    from oracle.flce_oracle import flce_oracle

    lib = emu_lib.EmuLib()                       # the library's kernels on the host (see tests/emu_lib.py)
    for mod in (fl, ce, sh):
        mod.lib = lib
    fl._stream = lambda device: None
    fl._device_guard = lambda device: contextlib.nullcontext()
    fl._require_cuda = lambda t: None
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        N, H, V = 300, 40, 203                   # two token chunks of the emulation's 256 rows
        x = torch.randn(N, H, generator=g).bfloat16()
        w = (torch.randn(V, H, generator=g) * 0.3).bfloat16()
        t = torch.randint(0, V, (N,), generator=g)
        t[::6] = -100
        ora = flce_oracle(x, w, t, **kw)

        def close(got, want, rtol=5e-2):
            got, want = got.double(), want.double()
            return bool(((got - want).abs() <= 8e-3 * float(want.abs().max()) + rtol * want.abs()).all())

        if mode == "token":
            lo, hi = rank * N // world, (rank + 1) * N // world
            xs, ws = x[lo:hi].clone().requires_grad_(True), w.clone().requires_grad_(True)
            loss = sh.token_sharded_fused_linear_cross_entropy(xs, ws, t[lo:hi], **kw)
            loss.backward()
            ok = abs(float(loss) - float(ora.loss)) <= 1e-4 * abs(float(ora.loss))
            ok &= close(xs.grad, ora.grad_input[lo:hi]) and close(ws.grad, ora.grad_weight)
        else:
            bounds = [0, 77, V]
            lo, hi = bounds[rank], bounds[rank + 1]
            xs, ws = x.clone().requires_grad_(True), w[lo:hi].clone().requires_grad_(True)
            loss = sh.vocab_sharded_fused_linear_cross_entropy(xs, ws, t, lo, V, **kw)
            loss.backward()
            ok = abs(float(loss) - float(ora.loss)) <= 1e-4 * abs(float(ora.loss))
            ok &= close(xs.grad, ora.grad_input) and close(ws.grad, ora.grad_weight[lo:hi])
        ok &= "flce_b200_forward_backward" in lib.calls and "flce_b200_backward" not in lib.calls
        with open(f"{result_file}.{rank}", "w") as f:
            f.write("ok" if ok else f"mismatch (store {getattr(lib, 'store_modes', None)})")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,kw", [
    ("token", dict()),
    ("token", dict(label_smoothing=0.1, lse_square_scale=1e-2)),
    ("vocab", dict()),
    ("vocab", dict(label_smoothing=0.1, lse_square_scale=1e-2)),
    ("vocab", dict(softcap=5.0, reduction="sum")),
    ("vocab", dict(softcap=5.0, label_smoothing=0.1)),          # smoothing under a soft-cap: the logits-store form
])
def test_two_ranks_form_gradients_in_forward_through_the_library_host_path(mode, kw):
    """16-bit operands, mean / sum: both sharded operators call the single-sweep entry point; the normalisers, the
    reference points, the per-chunk row statistics and the partial grad_input rows cross the ranks from inside it."""
    world = 2
    with tempfile.TemporaryDirectory() as tmp:
        init_file = os.path.join(tmp, "rendezvous")
        result = os.path.join(tmp, "result")
        mp.spawn(_emulated_worker, args=(world, init_file, mode, kw, result), nprocs=world, join=True)
        for r in range(world):
            with open(f"{result}.{r}") as f:
                assert f.read() == "ok", f"rank {r}"
