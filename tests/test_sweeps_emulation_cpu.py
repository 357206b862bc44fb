"""The two tensor-core sweeps of the fused linear cross-entropy at tile level on the CPU: the register epilogues
(csrc/epilogues.cuh: softmax statistics, logit gradient, store / accumulate) and the row kernels around them are the
library's own code compiled for the host; only the tcgen05 main loop is replaced, by a float dot product of the same
16-bit operands (tests/emu/emu_kernels.cpp::run_tiles).  The pipeline below strings them together in the order
flce_b200_forward / flce_b200_backward do and checks the result against the fp64 oracle and the reference's golden
vectors, so every feature of the hot path's arithmetic (bias, soft-cap and its chain rule, label smoothing, z-loss, class
weights, token scaling, ignore_index, reductions, upstream gradients, vocabulary shards, ragged shapes) is exercised on
every CPU run.  What this cannot see is the main loop itself (TMA, tensor memory, barriers): that is the GPU tests' job."""

import numpy as np
import pytest
import torch

import emu_lib
from flce_cases import assert_close, make_inputs, oracle_for
from golden_util import golden_grad_output, golden_kwargs, golden_names, load_golden

FMT = {torch.bfloat16: 0, torch.float16: 1}


@pytest.fixture(scope="module")
def emu():
    return emu_lib.load()


def _p(t):
    return None if t is None else t.data_ptr()


def flce_on_emulated_tiles(emu, x, w, t, bias=None, ce_weight=None, ignore_index=-100, lse_square_scale=0.0, label_smoothing=0.0,
                           reduction="mean", softcap=None, use_token_scaling=False, grad_output=None, vocab_offset=0,
                           vocab_total=None):
    """count -> sweep 1 -> merge -> finalize -> coefficients -> sweep 2 -> projections (the projections are plain matrix
    products of the 16-bit slab here).  Returns a dict shaped like flce_cases.run_cuda's."""
    dtype = x.dtype
    N, H = x.shape
    V = w.shape[0]
    vocab_total = V if vocab_total is None else vocab_total
    x, w, t = x.contiguous(), w.contiguous(), t.contiguous()
    bias32 = None if bias is None else bias.float().contiguous()
    cw = None if ce_weight is None else ce_weight.float().contiguous()
    cap = 0.0 if softcap is None else float(softcap)
    norm = torch.zeros(4)
    emu.emu_count(_p(t), N, ignore_index, _p(cw), V, vocab_offset, float(vocab_total), _p(norm))
    n_tiles = (V + 255) // 256
    planes = [torch.zeros(n_tiles, N) for _ in range(4)]
    pidx = torch.zeros(n_tiles, N, dtype=torch.int32)
    rowstats = torch.zeros(6, N)
    emu.emu_sweep_stats(_p(x), _p(w), FMT[dtype], N, V, H, x.stride(0), w.stride(0), _p(t), _p(bias32), _p(cw), cap, vocab_offset,
                        _p(planes[0]), _p(planes[1]), _p(planes[2]), _p(planes[3]), _p(pidx), rowstats[2].data_ptr(), None, 0, 0, -1, None, 0)
    emu.emu_merge_partials(N, n_tiles, _p(planes[0]), _p(planes[1]), _p(planes[2]), _p(planes[3]), _p(pidx), _p(rowstats))
    f = lambda: torch.zeros(N)                                                    # noqa: E731
    lse, prob, loss_rows, z_rows, correct = f(), f(), f(), f(), f()
    pred = torch.zeros(N, dtype=torch.int64)
    scalars = torch.zeros(4)
    mean = int(reduction == "mean")
    emu.emu_finalize(N, ignore_index, label_smoothing, lse_square_scale, mean, int(use_token_scaling), V, vocab_total, vocab_offset,
                     _p(t), _p(cw), _p(rowstats), _p(norm), _p(lse), _p(prob), _p(loss_rows), _p(z_rows), _p(correct), _p(pred),
                     _p(scalars))
    go = None
    per_row = 0
    if grad_output is not None:
        go = torch.as_tensor(grad_output, dtype=torch.float32).reshape(-1).contiguous()
        per_row = int(go.numel() == N and reduction == "none")
    c1, c2, c3 = f(), f(), f()
    emu.emu_coef(N, ignore_index, label_smoothing, lse_square_scale, mean, int(use_token_scaling), V, vocab_total, vocab_offset, _p(t),
                 _p(cw), _p(lse), _p(prob), _p(norm), _p(go), per_row, _p(c1), _p(c2), _p(c3))
    ld = (V + 63) // 64 * 64
    dz = torch.full((N, ld), 7.0).to(dtype)                                      # the padding must never be read back
    emu.emu_sweep_dz(_p(x), _p(w), FMT[dtype], N, V, H, x.stride(0), w.stride(0), _p(t), _p(bias32), _p(cw), cap, vocab_offset,
                     _p(lse), _p(c1), _p(c2), _p(c3), _p(dz), None, ld, FMT[dtype], -1)
    dzf = dz[:, :V].double()
    if reduction == "none":
        loss, z = loss_rows, z_rows
    else:
        loss, z = scalars[0], scalars[1]
    return dict(loss=loss, z_loss=z, lse=lse, token_accuracy=scalars[2], predicted_tokens=pred, grad_logits=dzf,
                grad_input=(dzf @ w.double()).to(dtype), grad_weight=(dzf.T @ x.double()).to(dtype),
                grad_bias=None if bias is None else dzf.sum(0).to(dtype), norm=norm, rowstats=rowstats)


def _check(res, ora, t, ignore_index=-100):
    scale = max(1.0, float(ora.loss.abs().max()))
    assert_close(res["loss"], ora.loss.float(), 1e-4 * scale, 1e-4, "loss")
    assert_close(res["z_loss"], ora.z_loss.float(), 2e-2 * max(1e-3, float(ora.z_loss.abs().max())), 1e-2, "z_loss")
    live = t != ignore_index
    assert_close(res["lse"][live], ora.lse.float()[live], 1e-5 * max(1.0, float(ora.lse.abs().max())), 1e-5, "lse")
    assert torch.equal(res["predicted_tokens"], ora.predicted_tokens)
    for key, want in (("grad_input", ora.grad_input), ("grad_weight", ora.grad_weight), ("grad_bias", ora.grad_bias)):
        if want is None:
            continue
        atol = 8e-3 * max(float(want.abs().max()), 1e-30)       # one 16-bit ulp of the tensor's largest entry, whatever its scale
        assert_close(res[key].float(), want.float(), atol, 5e-2, key)
    if bool((~live).any()):
        assert float(res["grad_input"][~live].abs().max()) == 0.0 and float(res["grad_logits"][~live].abs().max()) == 0.0


FEATURES = [dict(), dict(label_smoothing=0.1), dict(lse_square_scale=1e-4), dict(softcap=30.0),
            dict(label_smoothing=0.1, ignore_index=42, lse_square_scale=1e-4, softcap=30.0), dict(reduction="sum", softcap=5.0)]


@pytest.mark.parametrize("N,H,V", [(140, 64, 700), (47, 31, 123)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("feat", FEATURES)
def test_sweeps_match_oracle(emu, N, H, V, dtype, feat):
    x, w, t, b, _ = make_inputs(N, H, V, dtype, seed=N + V, bias=(H == 31), ignore_index=feat.get("ignore_index", -100))
    res = flce_on_emulated_tiles(emu, x, w, t, bias=b, **feat)
    _check(res, oracle_for(x, w, t, bias=b, **feat), t, feat.get("ignore_index", -100))


def test_sweeps_class_weights_token_scaling_and_upstream_gradients(emu):
    x, w, t, b, cw = make_inputs(96, 48, 203, torch.bfloat16, seed=3, bias=True, ce_weight=True)
    for kw, go in ((dict(label_smoothing=0.1), None), (dict(reduction="sum"), 2.5), (dict(reduction="none"), torch.rand(96) + 0.5)):
        res = flce_on_emulated_tiles(emu, x, w, t, bias=b, ce_weight=cw, grad_output=go, **kw)
        _check(res, oracle_for(x, w, t, bias=b, ce_weight=cw, grad_output=go, **kw), t)
    res = flce_on_emulated_tiles(emu, x, w, t, use_token_scaling=True)
    _check(res, oracle_for(x, w, t, use_token_scaling=True), t)
    # all rows ignored: exact zeros everywhere, no NaN from the empty normaliser
    t_all = torch.full_like(t, -100)
    res = flce_on_emulated_tiles(emu, x, w, t_all)
    assert float(res["loss"]) == 0.0 and float(res["grad_logits"].abs().max()) == 0.0 and bool((res["predicted_tokens"] == -1).all())


def test_sweeps_on_a_vocabulary_shard_merge_to_the_full_problem(emu):
    """Two shards of the vocabulary (global class ids, local columns): per-shard statistics merged as the vocab-sharded
    operator merges them give the full problem's lse and arg-max; the shard's logit gradient is the matching column block."""
    from liger_kernel_b200.sharded import merge_rowstats

    x, w, t, _, _ = make_inputs(70, 32, 400, torch.bfloat16, seed=8)
    full = flce_on_emulated_tiles(emu, x, w, t, label_smoothing=0.1)
    cut = 144
    shards = [flce_on_emulated_tiles(emu, x, w[:cut].contiguous(), t, label_smoothing=0.1, vocab_offset=0, vocab_total=400),
              flce_on_emulated_tiles(emu, x, w[cut:].contiguous(), t, label_smoothing=0.1, vocab_offset=cut, vocab_total=400)]
    merged = merge_rowstats(torch.stack([s["rowstats"] for s in shards]))
    lse = merged[0] + torch.log(merged[1])
    live = t != -100
    assert_close(lse[live], full["lse"][live], 1e-5, 1e-6, "merged lse")
    assert torch.equal(merged[5].view(torch.int32)[live].long(), full["predicted_tokens"][live])
    np.testing.assert_allclose(merged[2].numpy(), full["rowstats"][2].numpy(), rtol=0, atol=0)      # target logit: owner's value


@pytest.mark.parametrize("name", [n for n in golden_names() if load_golden(n)[1].get("dtype") == "bfloat16"] + ["mean_default", "all_features",
                                  "ce_weight", "token_scaling", "none_reduction", "grad_output_2p5"])
def test_sweeps_against_reference_golden(emu, name):
    """fp32 golden cases are fed as bf16 here (the sweeps take 16-bit operands), so they are compared through the oracle
    on the same rounded inputs; the bf16 golden case is compared with the reference's own outputs directly."""
    rec, meta = load_golden(name)
    bf16 = meta.get("dtype") == "bfloat16"
    x, w, t = (torch.from_numpy(rec[k]) for k in ("x", "w", "target"))
    x, w = x.bfloat16(), w.bfloat16()
    kw = golden_kwargs(rec, meta)
    if kw["bias"] is not None:
        kw["bias"] = kw["bias"].bfloat16()
    go = golden_grad_output(rec, meta)
    res = flce_on_emulated_tiles(emu, x, w, t, grad_output=go, **kw)
    _check(res, oracle_for(x, w, t, grad_output=go, **kw), t, meta["ignore_index"])
    if bf16:
        assert_close(res["loss"], torch.from_numpy(rec["ref_loss"]), 2e-2, 2e-2, "loss vs reference")
        want = torch.from_numpy(rec["ref_grad_weight"])
        assert_close(res["grad_weight"].float(), want, 1e-2 * float(want.abs().max()), 5e-2, "grad_weight vs reference")


@pytest.mark.parametrize("n", [256, 123, 8, 33])
def test_store_epilogue_ragged_columns_and_accumulator(emu, n):
    """D = A.B^T through StoreEpilogue for column counts that are not multiples of 8 or 32 (flce_b200_gemm_accumulate relies
    on the partial 16-byte groups staying inside the row pitch), 16-bit and fp32 outputs, with and without accumulator."""
    g = torch.Generator().manual_seed(n)
    m, k = 130, 40
    a = torch.randn(m, k, generator=g).bfloat16()
    b = torch.randn(n, k, generator=g).bfloat16()
    want = a.double() @ b.double().T
    ld = (n + 7) // 8 * 8 + 8
    for out_dtype, fmt in ((torch.bfloat16, 0), (torch.float32, 2)):
        out = torch.full((m + 1, ld), 3.0).to(out_dtype)                          # one guard row, guard columns
        emu.emu_gemm_store(_p(a), _p(b), 0, m, n, k, k, k, None, 0, _p(out), ld, fmt)
        assert_close(out[:m, :n].float(), want.float(), 1e-4, 2 ** -8 if fmt == 0 else 1e-6, "out")
        assert float((out[m] - 3.0).abs().max()) == 0.0                          # rows beyond M untouched
        assert float((out[:m, (n + 7) // 8 * 8:] - 3.0).abs().max()) == 0.0      # nothing written past the last 16-byte group
    acc = torch.ones(m, ld)
    emu.emu_gemm_store(_p(a), _p(b), 0, m, n, k, k, k, _p(acc), ld, None, 0, 2)
    emu.emu_gemm_store(_p(a), _p(b), 0, m, n, k, k, k, _p(acc), ld, None, 0, 2)
    assert_close(acc[:, :n], (1.0 + 2.0 * want).float(), 1e-4, 1e-6, "accumulator after two passes")
    assert float((acc[:, (n + 3) // 4 * 4:] - 1.0).abs().max()) == 0.0
