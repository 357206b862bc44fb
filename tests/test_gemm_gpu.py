"""The tcgen05 main loop in isolation, through the C ABI (flce_b200_gemm), against torch matmul.

Inputs are small integers, so every product and partial sum is exact in fp32 and the comparison
is bit-exact for every operand layout (K-major / MN-major) and for single CTAs and CTA pairs.
"""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

VARIANTS = [(0, 0), (0, 1), (1, 1), (1, 0)]  # (A MN-major?, B MN-major?): logits / dX / dW / dW against a transposed X
SHAPES = [(128, 256, 64), (256, 512, 256), (1000, 1304, 520), (136, 8, 72), (2048, 4096, 1024)]


def _run(a_mn, b_mn, pair, M, N, K, dtype=torch.bfloat16, out_dtype=torch.float32):
    from liger_kernel_b200 import _lib

    lib = _lib.lib
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    A = torch.randint(-3, 4, (M, K), device="cuda", generator=g).to(dtype)
    B = torch.randint(-3, 4, (N, K), device="cuda", generator=g).to(dtype)
    As = A.t().contiguous() if a_mn else A
    Bs = B.t().contiguous() if b_mn else B
    D = torch.full((M, N), float("nan"), device="cuda", dtype=out_dtype)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    code = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
    _lib.check(lib.flce_b200_gemm(C.c_void_p(As.data_ptr()), C.c_void_p(Bs.data_ptr()), C.c_void_p(D.data_ptr()),
                                  M, N, K, As.stride(0), Bs.stride(0), D.stride(0), code[dtype], code[out_dtype],
                                  a_mn, b_mn, pair, st))
    _lib.check(lib.flce_b200_check_device_status(st))
    ref = A.float() @ B.float().t()
    return D, ref


@pytest.mark.parametrize("pair", [0, 1])
@pytest.mark.parametrize("a_mn,b_mn", VARIANTS)
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_exact(M, N, K, a_mn, b_mn, pair):
    D, ref = _run(a_mn, b_mn, pair, M, N, K)
    assert torch.equal(D, ref), f"{int((D != ref).sum())} of {D.numel()} entries differ"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gemm_16bit_output(dtype):
    D, ref = _run(0, 0, 0, 300, 264, 136, dtype=dtype, out_dtype=dtype)
    assert torch.equal(D.float(), ref.to(dtype).float())


# K >= 2048 and N >= 1024 with CTA pairs select the 256 x 512 tile (two MMAs per K slice, one accumulator stage)
WIDE_SHAPES = [(256, 1024, 2048), (296, 1032, 2056), (1000, 1304, 2120), (2048, 4096, 2048), (520, 2560, 4160)]


@pytest.mark.parametrize("a_mn,b_mn", VARIANTS)
@pytest.mark.parametrize("M,N,K", WIDE_SHAPES)
def test_gemm_wide_tiles_exact(M, N, K, a_mn, b_mn):
    from liger_kernel_b200 import _lib

    D, ref = _run(a_mn, b_mn, 1, M, N, K)
    assert torch.equal(D, ref), f"{int((D != ref).sum())} of {D.numel()} entries differ"
    _lib.set_option("wide_tiles", 0)
    try:
        D2, _ = _run(a_mn, b_mn, 1, M, N, K)
    finally:
        _lib.set_option("wide_tiles", 1)
    assert torch.equal(D2, ref)


def test_gemm_wide_tiles_accumulate_across_calls():
    """fp32 partial results carried from call to call (the weight gradient over token chunks) with the wide tile."""
    from liger_kernel_b200 import _lib

    lib = _lib.lib
    M, N, K = 696, 1536, 2304
    g = torch.Generator(device="cuda").manual_seed(5)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    acc = torch.zeros((M, N), device="cuda", dtype=torch.float32)
    out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    ref = torch.zeros((M, N), device="cuda", dtype=torch.float32)
    for it in range(3):
        A = torch.randint(-2, 3, (K, M), device="cuda", generator=g).to(torch.bfloat16)      # MN-major, as dZ^T
        B = torch.randint(-2, 3, (K, N), device="cuda", generator=g).to(torch.bfloat16)      # MN-major, as X
        _lib.check(lib.flce_b200_gemm_accumulate(C.c_void_p(A.data_ptr()), C.c_void_p(B.data_ptr()), C.c_void_p(acc.data_ptr()),
                                                 C.c_void_p(out.data_ptr()), M, N, K, A.stride(0), B.stride(0), acc.stride(0),
                                                 out.stride(0), 0, 0, 1, 1, 1, st))
        ref += A.float().t() @ B.float()
    _lib.check(lib.flce_b200_check_device_status(st))
    assert torch.equal(acc, ref)
    assert torch.equal(out.float(), ref.bfloat16().float())


@pytest.mark.parametrize("stagger", [0, 25, 100])
@pytest.mark.parametrize("M,N,K", [(2048, 2048, 4096), (8192, 4096, 2048), (1000, 1304, 2120)])
def test_gemm_accumulate_with_staggered_first_tiles(M, N, K, stagger):
    """Running fp32 sum only (no 16-bit copy): partial products are added at L2, and every CTA pair cuts its first tile's K
    range in two at its own point so that the pairs' epilogues do not all hit memory at once.  Exact for small integers,
    whatever the cut (none, spread over a quarter of K, over all of K)."""
    from liger_kernel_b200 import _lib

    lib = _lib.lib
    g = torch.Generator(device="cuda").manual_seed(M + K)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    acc = torch.zeros((M, N), device="cuda", dtype=torch.float32)
    ref = torch.zeros((M, N), device="cuda", dtype=torch.float32)
    _lib.set_option("stagger_pct", stagger)
    try:
        for it in range(2):
            A = torch.randint(-2, 3, (K, M), device="cuda", generator=g).to(torch.bfloat16)
            B = torch.randint(-2, 3, (K, N), device="cuda", generator=g).to(torch.bfloat16)
            _lib.check(lib.flce_b200_gemm_accumulate(C.c_void_p(A.data_ptr()), C.c_void_p(B.data_ptr()), C.c_void_p(acc.data_ptr()),
                                                     None, M, N, K, A.stride(0), B.stride(0), acc.stride(0), 0, 0, 0, 1, 1, 1, st))
            ref += A.float().t() @ B.float()
    finally:
        _lib.set_option("stagger_pct", 0)
    _lib.check(lib.flce_b200_check_device_status(st))
    assert torch.equal(acc, ref)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pair,M,N,K", [(1, 1000, 1304, 2120), (1, 296, 1032, 2056), (1, 200, 264, 136), (0, 300, 264, 136),
                                        (1, 2048, 4096, 2048)])
def test_gemm_store_through_tma_matches_plain_stores(pair, M, N, K, out_dtype):
    """The store epilogue writes each 32 x 32 patch with one TMA store from shared memory (ragged edges clipped by the
    tensor map); with the option off it writes the same patch with ordinary vector stores.  Both exact."""
    from liger_kernel_b200 import _lib

    D, ref = _run(0, 1, pair, M, N, K, out_dtype=out_dtype)
    want = ref if out_dtype == torch.float32 else ref.to(out_dtype).float()
    assert torch.equal(D.float(), want)
    _lib.set_option("bulk_store", 0)
    try:
        D2, _ = _run(0, 1, pair, M, N, K, out_dtype=out_dtype)
    finally:
        _lib.set_option("bulk_store", 1)
    assert torch.equal(D2.float(), want)
