"""flce_b200_forward_stats_static: the forward-statistics sweep for callers that cannot allocate device memory
(a host with a fixed memory plan, a latency-critical loop).  Its scratch is a 32 MiB array inside the library.
Called through the C ABI and compared with flce_b200_forward_stats (caller-provided workspace) on the same
inputs: the two run the same kernels on differently placed scratch, so the statistics must be identical; the
log-sum-exp they imply is also checked against the CPU oracle.  Two calls in a row with different shapes check that
contents left behind by the first do not leak into the second.  "Allocates nothing" is checked two ways: torch's
allocator counter, and the free device memory the CUDA runtime reports (which would see a cudaMalloc inside the library).
This file is named to be collected last."""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(N, H, V, seed, **kw):
    from liger_kernel_b200 import _lib
    from liger_kernel_b200.ops.fused_linear_cross_entropy import _Prepared, _ptr, _stream

    lib = _lib.lib
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(N, H, generator=g, device="cuda").bfloat16()
    w = (torch.randn(V, H, generator=g, device="cuda") * 0.05).bfloat16()
    t = torch.randint(0, V, (N,), generator=g, device="cuda")
    t[::11] = -100
    prep = _Prepared(x, w, t, None, None, -100, 0.0, kw.get("label_smoothing", 0.0), "mean", kw.get("softcap"), False,
                     want_argmax=kw.get("want_argmax", False))
    ws = prep.workspace(_lib.PHASE_FORWARD)
    ref = torch.full((_lib.ROWSTAT_PLANES, N), float("nan"), device="cuda")
    got = torch.full((_lib.ROWSTAT_PLANES, N), float("nan"), device="cuda")
    _lib.check(lib.flce_b200_forward_stats(C.byref(prep.problem), _ptr(ref), _ptr(ws), ws.numel(), _stream(x.device)))
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before, _ = torch.cuda.mem_get_info()
    _lib.check(lib.flce_b200_forward_stats_static(C.byref(prep.problem), _ptr(got), _stream(x.device)))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_allocated() == before
    if _both.warm:       # (the very first call on a device may make the runtime load the kernel's module)
        assert free_after == free_before, (free_before, free_after)
    _both.warm = True
    _lib.check(lib.flce_b200_check_device_status(_stream(x.device)))
    # the statistics against the oracle: lse = max + log(sum exp) per row, to 1e-5
    from oracle.flce_oracle import flce_oracle

    ora = flce_oracle(x.cpu(), w.cpu(), t.cpu(), label_smoothing=kw.get("label_smoothing", 0.0), softcap=kw.get("softcap"))
    lse = (got[0] + torch.log(got[1])).double().cpu()
    valid = (t != -100).cpu()          # (the oracle reports 0 on ignored rows)
    err = ((lse - ora.lse).abs() / ora.lse.abs().clamp(min=1.0))[valid].max()
    assert float(err) <= 1e-5, float(err)
    return ref, got, kw.get("want_argmax", False)


_both.warm = False


def _same(ref, got, with_argmax):
    planes = [0, 1, 2, 3] + ([4, 5] if with_argmax else [])
    for i in planes:
        assert torch.equal(ref[i].view(torch.int32), got[i].view(torch.int32)), f"plane {i} differs"


def test_static_scratch_matches_workspace_variant_twice_in_a_row():
    # first call: all optional planes in use, ragged shapes
    _same(*_both(1000, 264, 5003, seed=1, label_smoothing=0.1, softcap=20.0, want_argmax=True))
    # second call right after, smaller and with fewer planes: stale scratch contents must not matter
    _same(*_both(300, 128, 1000, seed=2))
    # and once more with the first shape: the array is reused as is
    _same(*_both(1000, 264, 5003, seed=3, label_smoothing=0.1, want_argmax=True))


def test_static_scratch_rejects_oversized_problem():
    from liger_kernel_b200 import _lib
    from liger_kernel_b200.ops.fused_linear_cross_entropy import _Prepared, _ptr, _stream

    N, H, V = 8192, 64, 400000       # 2 planes x 1563 tiles x 8192 rows > 8 Mi floats
    x = torch.zeros(N, H, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(V, H, device="cuda", dtype=torch.bfloat16)
    t = torch.zeros(N, device="cuda", dtype=torch.long)
    prep = _Prepared(x, w, t, None, None, -100, 0.0, 0.0, "mean", None, False, want_argmax=False)
    out = torch.empty((_lib.ROWSTAT_PLANES, N), device="cuda")
    rc = _lib.lib.flce_b200_forward_stats_static(C.byref(prep.problem), _ptr(out), _stream(x.device))
    assert rc == 3
    msg = _lib.lib.flce_b200_last_error().decode()
    assert "too large for the built-in scratch" in msg and "32 MiB" in msg
