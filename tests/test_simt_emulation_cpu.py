"""The library's SIMT kernels (everything outside the tensor-core sweeps) compiled for the host and run on the host
(tests/emu/): real numerics on CPU for the stand-alone cross-entropy operator, target counting, row compaction and
scatter, the fp32 term split, the single-sweep mode's in-place logit gradient, column sums and gradient scaling.

ex2.approx / rcp.approx are libm calls here, so agreement with the GPU is to a few ulp; the checks are against the fp64
oracle and exact numpy restatements with the GPU tests' tolerances.  The stand-alone cross-entropy cases are the GPU
test's own bodies (tests/ce_cases.py) at smaller row counts."""

import ctypes as C

import numpy as np
import pytest
import torch

import ce_cases
import emu_lib
from golden_util import ce_golden_names


@pytest.fixture(scope="module")
def emu():
    return emu_lib.load()


# ---------------------------------------------------------------- stand-alone cross-entropy through the Python operator
CE_GRID = [(19, 123, dt, red, f) for dt in (torch.bfloat16, torch.float16, torch.float32) for red in ("mean", "sum")
           for f in range(len(ce_cases.FEATURES))]
CE_GRID += [(24, 4096, dt, "mean", f) for dt in (torch.bfloat16, torch.float32) for f in (0, 4)]
CE_GRID += [(3, 128256, torch.bfloat16, "mean", 4), (3, 128256, torch.float32, "sum", 1), (5, 32001, torch.float16, "mean", 4),
            (5, 32001, torch.float32, "mean", 3)]


@pytest.mark.parametrize("N,V,dtype,reduction,feat", CE_GRID)
def test_ce_correctness(monkeypatch, N, V, dtype, reduction, feat):
    with emu_lib.installed(monkeypatch):
        ce_cases.case_correctness("cpu", N, V, dtype, reduction, ce_cases.FEATURES[feat])


def test_ce_weights_none_reduction_upstream_gradient_and_inplace(monkeypatch):
    with emu_lib.installed(monkeypatch):
        ce_cases.case_weights_none_reduction_upstream_gradient_and_inplace("cpu", N=40, V=1000)


def test_ce_all_ignored_is_exact_zero(monkeypatch):
    with emu_lib.installed(monkeypatch):
        ce_cases.case_all_ignored_is_exact_zero("cpu", N=9, V=500)


@pytest.mark.parametrize("name", ce_golden_names())
def test_ce_against_reference_golden(monkeypatch, name):
    with emu_lib.installed(monkeypatch):
        ce_cases.case_reference_golden("cpu", name)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("label_smoothing,reduction", [(0.0, "mean"), (0.1, "sum")])
def test_ce_true_class_gradient_confident_predictions(monkeypatch, dtype, label_smoothing, reduction):
    with emu_lib.installed(monkeypatch):
        ce_cases.case_true_class_gradient_confident_predictions("cpu", dtype, label_smoothing, reduction)


def test_ce_forward_only_structured_output_and_target_check(monkeypatch):
    with emu_lib.installed(monkeypatch):
        ce_cases.case_forward_only_structured_output_and_target_check("cpu")


def test_ce_rows_with_minus_inf_and_unaligned_views(monkeypatch):
    """-inf logits (masked classes) keep the statistics finite; a column-sliced view (row pitch not a multiple of 16
    bytes, base not 16-byte aligned) takes the scalar kernels and gives the same answer as the vectorised ones."""
    from oracle.flce_oracle import ce_oracle

    g = torch.Generator().manual_seed(5)
    full = torch.randn(6, 211, generator=g) * 2
    full[:, 7] = float("-inf")
    full[2, :100] = float("-inf")
    t = torch.tensor([0, 5, 150, 210, -100, 3])
    with emu_lib.installed(monkeypatch):
        for dtype in (torch.float32, torch.bfloat16):
            wide = torch.zeros(6, 216).to(dtype)
            wide[:, 3:214] = full.to(dtype)
            view = wide[:, 3:214]                                  # pitch 216, offset 3 elements: not vectorisable
            assert view.data_ptr() % 16 != 0
            dense = full.to(dtype).contiguous()
            ora = ce_oracle(dense, t, label_smoothing=0.0)
            a = ce_cases.run_ce(dense, t, "cpu")
            b = ce_cases.run_ce(view, t, "cpu")
            ce_cases.check_ce(a, ora, dtype)
            assert torch.equal(a["predicted"], b["predicted"])
            np.testing.assert_allclose(a["loss"].numpy(), b["loss"].numpy(), rtol=1e-6)
            np.testing.assert_allclose(a["grad"].numpy(), b["grad"].numpy(), rtol=1e-5, atol=1e-8)
            assert np.isfinite(a["grad"].numpy()).all()


# ---------------------------------------------------------------- target counting
@pytest.mark.parametrize("n", [1, 31, 1024, 2500])
def test_count_kernel(emu, n):
    g = np.random.default_rng(n)
    V, off, total = 40, 16, 100
    t = g.integers(0, total, n).astype(np.int64)
    t[g.random(n) < 0.2] = -100
    if n > 3:
        t[1], t[2] = 100, -5                                           # outside [0, total): counted, never dereferenced
    w = (g.random(V) + 0.5).astype(np.float32)
    for weight in (None, w):
        norm = np.zeros(4, np.float32)
        emu.emu_count(t.ctypes.data, n, -100, None if weight is None else weight.ctypes.data, V, off, float(total),
                      norm.ctypes.data)
        live = t != -100
        assert norm[0] == live.sum() and norm[3] == (live & ((t < 0) | (t >= total))).sum()
        if weight is None:
            assert norm[1] == live.sum() and norm[2] == total
        else:
            local = t[live] - off
            inside = local[(local >= 0) & (local < V)]
            np.testing.assert_allclose(norm[1], w[inside].astype(np.float64).sum(), rtol=1e-5)
            np.testing.assert_allclose(norm[2], w.astype(np.float64).sum(), rtol=1e-5)


# ---------------------------------------------------------------- row compaction and scatter
@pytest.mark.parametrize("n,frac", [(1, 0.0), (1, 1.0), (5, 0.5), (1023, 0.3), (1024, 0.9), (1025, 0.5), (3000, 0.05), (2048, 0.0),
                                    (2049, 1.0)])
def test_compact_and_scatter_rows(emu, n, frac):
    g = np.random.default_rng(n)
    hidden, ld = 24, 40
    x = g.integers(0, 65536, (n, ld)).astype(np.uint16)
    t = g.integers(0, 50, n).astype(np.int64)
    t[g.random(n) < frac] = -100
    if frac == 1.0:
        t[:] = -100
    xc = np.zeros((n, hidden), np.uint16)
    tc = np.zeros(n, np.int64)
    perm = np.full(n, -1, np.int32)
    active = np.zeros(1, np.int32)
    emu.emu_compact_rows(x.ctypes.data, ld, hidden, n, t.ctypes.data, -100, xc.ctypes.data, tc.ctypes.data, perm.ctypes.data,
                         active.ctypes.data)
    live, rest = np.nonzero(t != -100)[0], np.nonzero(t == -100)[0]
    want = np.concatenate([live, rest])
    assert active[0] == len(live)
    assert np.array_equal(perm, want)                                      # stable: both groups keep token order
    assert np.array_equal(xc, x[want, :hidden]) and np.array_equal(tc, t[want])
    # scatter a per-row result back: live rows return to their tokens, ignored tokens read exact zeros
    src = g.integers(1, 255, (n, 32)).astype(np.uint8)
    dst = np.full((n, 32), 0xEE, np.uint8)
    emu.emu_scatter_rows(src.ctypes.data, 32, perm.ctypes.data, active.ctypes.data, n, dst.ctypes.data)
    back = np.zeros((n, 32), np.uint8)
    back[want[:len(live)]] = src[:len(live)]
    assert np.array_equal(dst, back)


# ---------------------------------------------------------------- fp32 -> bf16 term split
def test_split_fp32_terms_sum_back(emu):
    g = torch.Generator().manual_seed(0)
    rows, cols, block = 7, 21, 24
    src = torch.randn(rows, cols, generator=g) * 3
    pattern = (0, 0, 0, 1, 1, 2)
    out = torch.full((rows, len(pattern) * block), 7.0).bfloat16()
    pat = (C.c_int * 8)(*pattern)
    emu.emu_split_fp32(src.data_ptr(), rows, cols, cols, out.data_ptr(), out.stride(0), block, C.addressof(pat), len(pattern), 0)
    t0 = src.bfloat16()
    t1 = (src - t0.float()).bfloat16()
    t2 = (src - t0.float() - t1.float()).bfloat16()
    terms = (t0, t1, t2)
    for b, k in enumerate(pattern):
        blk = out[:, b * block:(b + 1) * block]
        assert torch.equal(blk[:, :cols], terms[k]) and float(blk[:, cols:].abs().max()) == 0.0
    err = (t0.double() + t1.double() + t2.double() - src.double()).abs().max()
    assert float(err) <= 2.0 ** -22 * float(src.abs().max())


def test_python_split_helper_on_the_emulation(monkeypatch):
    """_Prepared's fp32 path end to end on the host: six X term blocks and six W term blocks whose pairwise products
    sum to the fp32 dot product."""
    import liger_kernel_b200.ops.fused_linear_cross_entropy as fl

    with emu_lib.installed(monkeypatch):
        g = torch.Generator().manual_seed(1)
        x, w = torch.randn(5, 20, generator=g), torch.randn(9, 20, generator=g)
        xs = fl._split_fp32(x, fl._X_TERMS, 24)
        ws = fl._split_fp32(w, fl._W_TERMS, 24)
        got = xs.double() @ ws.double().T
        want = x.double() @ w.double().T
        assert float((got - want).abs().max()) < 3e-6 * float(want.abs().max())


# ---------------------------------------------------------------- single-sweep pieces
@pytest.mark.parametrize("fmt,softcap", [(0, 0.0), (1, 0.0), (0, 30.0)])
def test_dz_inplace_kernel(emu, fmt, softcap):
    g = torch.Generator().manual_seed(fmt + 1)
    rows, vocab, ld, off = 5, 2100, 2112, 1000                              # vocabulary shard starting at class 1000
    dt = torch.bfloat16 if fmt == 0 else torch.float16
    s = (torch.randn(rows, ld, generator=g) * 2).to(dt)                        # stored (soft-capped) logits
    t = torch.tensor([1000, 3099, 50, 2000, 1500])                            # global ids; 50 is outside the shard
    lse = torch.logsumexp(s[:, :vocab].float(), dim=1) + 0.3
    c1, c2, c3 = torch.rand(rows, generator=g) + 0.5, torch.rand(rows, generator=g) * 0.01, torch.rand(rows, generator=g)
    colw = torch.rand(vocab, generator=g) + 0.5
    sf = s[:, :vocab].double()
    want = torch.exp(sf - lse.double()[:, None]) * c1.double()[:, None] - c2.double()[:, None] * colw.double()[None, :]
    for r in range(rows):
        j = int(t[r]) - off
        if 0 <= j < vocab:
            want[r, j] -= float(c3[r])
    if softcap > 0:
        want = want * (1 - (sf / softcap) ** 2)
    slab = s.clone()
    emu.emu_dz_inplace(slab.data_ptr(), ld, rows, vocab, fmt, t.data_ptr(), off, lse.data_ptr(), c1.data_ptr(), c2.data_ptr(),
                       c3.data_ptr(), colw.data_ptr(), 1.0 / softcap if softcap > 0 else 0.0, None, 0)
    got = slab[:, :vocab].double()
    tol = 2.0 ** -8 if fmt == 0 else 2.0 ** -10
    assert float(((got - want).abs() - tol * want.abs()).max()) <= 1e-6
    assert float(slab[:, vocab:vocab // 8 * 8 + 8].abs().max()) == 0.0          # columns past the vocabulary in the last vector


def test_colsum_and_scale_and_merge(emu):
    g = torch.Generator().manual_seed(2)
    rows, cols, ld = 70, 130, 136
    dz = torch.randn(rows, ld, generator=g).bfloat16()
    out = torch.ones(cols)
    emu.emu_colsum(dz.data_ptr(), ld, rows, cols, 0, out.data_ptr(), 1, None, 0)
    np.testing.assert_allclose(out.numpy(), 1.0 + dz[:, :cols].float().sum(0).numpy(), rtol=1e-5, atol=1e-5)
    emu.emu_colsum(dz.data_ptr(), ld, rows, cols, 0, out.data_ptr(), 0, None, 0)
    np.testing.assert_allclose(out.numpy(), dz[:, :cols].float().sum(0).numpy(), rtol=1e-5, atol=1e-5)
    # scaling: bf16, fp32, and the no-op when the factor is exactly one
    for t, fmt in ((torch.randn(1000, generator=g).bfloat16(), 0), (torch.randn(1000, generator=g).half(), 1),
                   (torch.randn(1000, generator=g), 2)):
        for factor in (1.0, 0.37):
            data, scale = t.clone(), torch.tensor([factor])
            emu.emu_scale_inplace(data.data_ptr(), data.numel(), fmt, scale.data_ptr())
            assert torch.equal(data, (t.float() * factor).to(t.dtype))
    # merging per-tile softmax partials
    n, tiles = 37, 5
    pmax = torch.randn(tiles, n, generator=g)
    pmax[3] = float("-inf")                                                   # an all-masked tile
    psum = torch.rand(tiles, n, generator=g) + 0.1
    psum[3] = 0.0
    pls, pav = torch.randn(tiles, n, generator=g), torch.randn(tiles, n, generator=g)
    pai = torch.randint(0, 1000, (tiles, n), generator=g, dtype=torch.int32)
    rowstats = torch.zeros(6, n)
    emu.emu_merge_partials(n, tiles, pmax.data_ptr(), psum.data_ptr(), pls.data_ptr(), pav.data_ptr(), pai.data_ptr(),
                           rowstats.data_ptr())
    m = pmax.max(0).values
    np.testing.assert_array_equal(rowstats[0].numpy(), m.numpy())
    np.testing.assert_allclose(rowstats[1].numpy(), (psum * torch.exp(pmax - m)).sum(0).numpy(), rtol=1e-6)
    np.testing.assert_allclose(rowstats[3].numpy(), pls.sum(0).numpy(), rtol=1e-5, atol=1e-6)
    best = pav.argmax(0)
    assert torch.equal(rowstats[5].view(torch.int32), pai.gather(0, best[None])[0])


# ---------------------------------------------------------------- tile schedule of the tensor-core main loop
@pytest.mark.parametrize("m_tiles,n_tiles", [(1, 1), (3, 7), (128, 501), (501, 16), (64, 4), (37, 37)])
@pytest.mark.parametrize("num_units", [74, 148, 5])
def test_tile_schedule_visits_every_tile_once(emu, m_tiles, n_tiles, num_units):
    """The producer, the MMA issuer and the epilogue warps of a persistent CTA derive their tiles from the same arithmetic
    (csrc/tile_schedule.cuh); here: for every raster group shape the walk over all units reaches each tile exactly once, and
    consecutive tiles of a group share the operand panel the raster is meant to keep in L2."""
    for along_m in (0, 1):
        extent = m_tiles if along_m else n_tiles
        for group in sorted({1, 2, 3, 8, extent, max(1, extent - 1), extent + 5}):
            visits = np.zeros(m_tiles * n_tiles, np.int32)
            order = np.full(m_tiles * n_tiles, -1, np.int32)
            rc = emu.emu_tile_schedule(m_tiles, n_tiles, group, along_m, num_units, visits.ctypes.data, order.ctypes.data)
            assert rc == 0 and (visits == 1).all(), (m_tiles, n_tiles, group, along_m)
    # walk order inside the first group (one unit sees every tile): group of g m-tiles x all n-tiles, m fastest
    g = min(3, m_tiles)
    visits = np.zeros(m_tiles * n_tiles, np.int32)
    order = np.full(m_tiles * n_tiles, -1, np.int32)
    emu.emu_tile_schedule(m_tiles, n_tiles, g, 1, 1, visits.ctypes.data, order.ctypes.data)
    first = [(int(t) // n_tiles, int(t) % n_tiles) for t in order[:g * n_tiles]]
    assert first == [(m, n) for n in range(n_tiles) for m in range(g)]


def test_active_rows_shrink_m_tiles_or_k_blocks(emu):
    out = np.zeros(2, np.int32)

    def limit(m_tiles, k_blocks, role, rows, ctas):
        emu.emu_limit_to_active_rows(m_tiles, k_blocks, role, rows, ctas, out.ctypes.data)
        return int(out[0]), int(out[1])

    assert limit(100, 50, 0, 10, 1) == (100, 50)                       # no role: untouched
    assert limit(100, 50, 1, 0, 1) == (0, 50) and limit(100, 50, 2, 0, 2) == (100, 0)
    assert limit(100, 50, 1, 1, 1) == (1, 50) and limit(100, 50, 1, 128, 1) == (1, 50) and limit(100, 50, 1, 129, 1) == (2, 50)
    assert limit(100, 50, 1, 256, 2) == (1, 50) and limit(100, 50, 1, 257, 2) == (2, 50)      # a CTA pair owns 256 rows
    assert limit(100, 50, 2, 64, 1) == (100, 1) and limit(100, 50, 2, 65, 2) == (100, 2)
    assert limit(100, 50, 1, 10 ** 9, 1) == (100, 50) and limit(100, 50, 2, 10 ** 9, 1) == (100, 50)   # never grows
    assert limit(100, 50, 1, -5, 1) == (0, 50)                         # a negative count reads as zero
