"""Token-sharded and vocabulary-sharded FLCE on real GPUs (NCCL), one process per GPU, against the single-GPU
operator on the whole problem.  Skipped when fewer than two GPUs are visible (as the reference skips its
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
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from liger_kernel_b200 import sharded
    from liger_kernel_b200.ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction as Fn

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        notes = []

        def close(got, want, what, rtol=5e-2):
            # 16-bit gradients: compare relative to the tensor's scale (one bf16 ulp of the largest entry) plus rtol
            atol = 8e-3 * float(want.abs().max())
            bad = (got.float() - want.float()).abs() > atol + rtol * want.float().abs()
            notes.append(f"{what}: max|diff| {float((got.float() - want.float()).abs().max()):.3e} max|want| "
                         f"{float(want.abs().max()):.3e} bad {int(bad.sum())}")
            return not bool(bad.any())

        g = torch.Generator().manual_seed(17)
        N, H, V = 1024, 256, 5000
        x = torch.randn(N, H, generator=g).bfloat16().cuda()
        w = (torch.randn(V, H, generator=g) * 0.05).bfloat16().cuda()
        t = torch.randint(0, V, (N,), generator=g)
        t[::9] = -100
        t = t.cuda()
        xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        ref = Fn.apply(xr, wr, t, None, None, -100, kw.get("lse_square_scale", 0.0), kw.get("label_smoothing", 0.0),
                       kw.get("reduction", "mean"), kw.get("softcap"))[0]
        ref.backward()
        if mode == "token":
            lo, hi = rank * N // world, (rank + 1) * N // world
            xs, ws = x[lo:hi].clone().requires_grad_(True), w.clone().requires_grad_(True)
            import liger_kernel_b200.ops.fused_linear_cross_entropy as mod
            mod.SLAB_BUDGET_BYTES = (hi - lo) * 2 * 1024      # several slabs: exercises the overlapped all-reduce
            ok = True
            for overlap in (True, False):           # slab-by-slab all-reduce on a side stream / one all-reduce at the end (default)
                xs.grad = ws.grad = None
                loss = sharded.token_sharded_fused_linear_cross_entropy(xs, ws, t[lo:hi], overlap_grad_weight=overlap, **kw)
                loss.backward()
                ok &= close(loss, ref, f"loss overlap={overlap}", rtol=1e-5)
                ok &= close(xs.grad, xr.grad[lo:hi], f"grad_input overlap={overlap}")
                ok &= close(ws.grad, wr.grad, f"grad_weight overlap={overlap}")
        else:
            per = (V + world - 1) // world
            lo, hi = rank * per, min(V, (rank + 1) * per)
            xs, ws = x.clone().requires_grad_(True), w[lo:hi].clone().requires_grad_(True)
            loss = sharded.vocab_sharded_fused_linear_cross_entropy(xs, ws, t, lo, V, **kw)
            loss.backward()
            ok = close(loss, ref, "loss", rtol=1e-5)
            ok &= close(xs.grad, xr.grad, "grad_input")
            ok &= close(ws.grad, wr.grad[lo:hi], "grad_weight")
        torch.cuda.synchronize()
        with open(f"{result_file}.{rank}", "w") as f:
            f.write("ok" if bool(ok) else "mismatch: " + "; ".join(notes))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["token", "vocab"])
@pytest.mark.parametrize("kw", [dict(), dict(label_smoothing=0.1, lse_square_scale=1e-3, softcap=30.0, reduction="sum")])
def test_sharded_equals_single_gpu(mode, kw):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    with tempfile.TemporaryDirectory() as tmp:
        init_file, result = os.path.join(tmp, "rdv"), os.path.join(tmp, "res")
        mp.spawn(_worker, args=(world, init_file, mode, kw, result), nprocs=world, join=True)
        for r in range(world):
            with open(f"{result}.{r}") as f:
                assert f.read() == "ok", f"rank {r}"
