"""Token-sharded and vocabulary-sharded FLCE on real GPUs (NCCL), one process per GPU, against the CPU oracle of
the whole problem.  Skipped when fewer than two GPUs are visible (as the reference skips its
multi-GPU test, test/megatron/test_cross_entropy.py:691-715)."""

import os
import sys
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _worker(rank, world, init_file, mode, kw, result_file):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.join(os.path.dirname(HERE), "liger-kernel_b200"))
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from liger_kernel_b200 import sharded
    from oracle.flce_oracle import flce_oracle

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        notes = []

        def close(got, want, what, rtol=5e-2, atol_scale=8e-3):
            # 16-bit gradients: relative to the tensor's scale (one bf16 ulp of the largest entry) plus rtol;
            # the loss: 1e-4 relative, nothing absolute
            got, want = got.detach().double().cpu(), want.detach().double().cpu()
            atol = atol_scale * float(want.abs().max())
            bad = (got - want).abs() > atol + rtol * want.abs()
            notes.append(f"{what}: max|diff| {float((got - want).abs().max()):.3e} max|want| {float(want.abs().max()):.3e} "
                         f"bad {int(bad.sum())}")
            return not bool(bad.any())

        g = torch.Generator().manual_seed(17)
        N, H, V = 1024, 256, 5003          # V / world is never a multiple of the 256-column tile
        x = torch.randn(N, H, generator=g).bfloat16()
        w = (torch.randn(V, H, generator=g) * 0.05).bfloat16()
        t = torch.randint(0, V, (N,), generator=g)
        t[::9] = -100
        ora = flce_oracle(x, w, t, **kw)       # fp64 on the same 16-bit inputs
        x, w, t = x.cuda(), w.cuda(), t.cuda()
        ok = True
        if mode == "token":
            lo, hi = rank * N // world, (rank + 1) * N // world
            xs, ws = x[lo:hi].clone().requires_grad_(True), w.clone().requires_grad_(True)
            import liger_kernel_b200.ops.fused_linear_cross_entropy as mod
            mod.SLAB_BUDGET_BYTES = (hi - lo) * 2 * 1024      # several slabs: exercises the slab-by-slab all-reduce of the two-sweep path
            for overlap in (True, False):
                xs.grad = ws.grad = None
                loss = sharded.token_sharded_fused_linear_cross_entropy(xs, ws, t[lo:hi], overlap_grad_weight=overlap, **kw)
                if kw.get("reduction") == "none":
                    go = torch.linspace(0.5, 1.5, N)
                    loss.backward(go[lo:hi].cuda())
                    want = flce_oracle(x.cpu(), w.cpu(), t.cpu(), grad_output=go, **kw)
                    ok &= close(loss, want.loss[lo:hi], f"loss rows overlap={overlap}", rtol=1e-4, atol_scale=1e-5)
                else:
                    loss.backward()
                    want = ora
                    ok &= close(loss, want.loss, f"loss overlap={overlap}", rtol=1e-4, atol_scale=0.0)
                ok &= close(xs.grad, want.grad_input[lo:hi], f"grad_input overlap={overlap}")
                ok &= close(ws.grad, want.grad_weight, f"grad_weight overlap={overlap}")
        else:
            per = (V + world - 1) // world
            lo, hi = rank * per, min(V, (rank + 1) * per)
            xs, ws = x.clone().requires_grad_(True), w[lo:hi].clone().requires_grad_(True)
            loss = sharded.vocab_sharded_fused_linear_cross_entropy(xs, ws, t, lo, V, **kw)
            loss.backward()
            ok &= close(loss, ora.loss, "loss", rtol=1e-4, atol_scale=0.0)
            ok &= close(xs.grad, ora.grad_input, "grad_input")
            ok &= close(ws.grad, ora.grad_weight[lo:hi], "grad_weight")
        torch.cuda.synchronize()
        with open(f"{result_file}.{rank}", "w") as f:
            f.write("ok" if bool(ok) else "mismatch: " + "; ".join(notes))
    finally:
        dist.destroy_process_group()


CASES = [
    ("token", dict()),
    ("token", dict(label_smoothing=0.1, lse_square_scale=1e-3, softcap=30.0, reduction="sum")),
    ("token", dict(reduction="none")),
    ("vocab", dict()),
    ("vocab", dict(label_smoothing=0.1, lse_square_scale=1e-3, softcap=30.0, reduction="sum")),
]


@pytest.mark.parametrize("mode,kw", CASES)
def test_sharded_equals_oracle(mode, kw):
    """Every rank's loss (1e-4 relative) and gradients (16-bit bar) against the fp64 oracle of the whole problem, on as
    many GPUs as the box shows (up to 8)."""
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    with tempfile.TemporaryDirectory() as tmp:
        init_file, result = os.path.join(tmp, "rdv"), os.path.join(tmp, "res")
        mp.spawn(_worker, args=(world, init_file, mode, kw, result), nprocs=world, join=True)
        for r in range(world):
            with open(f"{result}.{r}") as f:
                assert f.read() == "ok", f"rank {r}"
